#!/usr/bin/env python
"""Headline benchmark: GLM-5-class NVFP4 decode throughput (tokens/s), tensor parallel over N GPUs.

`python bench.py --gpus N --steps K --warmup W`  (N > 1: launched under torch.distributed.run,
one rank per GPU).  Synthetic token ids, random-init NVFP4 weights of the GLM-5 architecture
(78 layers when they fit in N x 180 GB; otherwise the largest layer count that fits, named in
`config.layers`).  Prints ONE JSON line on rank 0.

value      : aggregate decode tokens/s at batch 8, MTP off, timed on the device with CUDA events
             around K CUDA-graph replays (max over ranks).
e2e.value  : the same K steps through the public `Engine.decode_step` API, each step copying
             its inputs host->device from pinned memory and reading the sampled tokens back.
details    : batch 1 decode, MTP=3 verification-step rates, prefill throughput;
             `fixed_layers`: the same decode step on the layer count that one GPU holds (a like-for-like 1 -> N curve);
             `batch8_prefix`: 8 requests x 8192-token prompts with a shared 4096-token prefix through the
             continuous-batching scheduler (aggregate decode tok/s, p50 time to first token; full model only);
             `prefill_128k_cp`: one 131072-token prompt under context parallelism (full model, N = 8 only).
Every rank checks that all ranks sampled the same tokens.
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import statistics
import subprocess
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

BASELINE_BS1_STEPS_S = 60.8       # reference, 8x RTX PRO 6000: verification steps/s at concurrency 1, MTP 3 (VLLM-bench.md:26)
BASELINE_BS8_STEPS_S = 163.5      # ... at concurrency 8
BASELINE_PREFILL_128K_TOK_S = 4638.0
FIXED_LAYERS = 28                 # layers of the like-for-like run: what one 180 GB GPU holds next to its KV cache


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (0 = as many as fit, up to 78)")
    ap.add_argument("--prompt-len", type=int, default=4096)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--mtp", type=int, default=3)
    ap.add_argument("--no-fused", action="store_true", help="use the NCCL collectives instead of the NVLink kernels")
    ap.add_argument("--skip-details", action="store_true")
    ap.add_argument("--skip-fixed", action="store_true", help="no like-for-like run on the one-GPU layer count")
    ap.add_argument("--skip-serving", action="store_true", help="no scheduler run (8 requests, shared prefix)")
    ap.add_argument("--skip-cp", action="store_true", help="no 128K context-parallel prefill run")
    ap.add_argument("--serving-decode", type=int, default=512, help="tokens each request of the scheduler run decodes")
    ap.add_argument("--cp-context", type=int, default=131072)
    ap.add_argument("--tiny", action="store_true", help="small model (smoke runs)")
    return ap.parse_args()


class ClockSampler:
    """Samples `nvidia-smi` clocks / throttle reasons of one GPU during the timed region."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.path = f"/tmp/slopllm_clocks_{os.getpid()}.csv"

    def start(self):
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=self.f,
                                         stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.f.close()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        os.unlink(self.path)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def layer_bytes(cfg, world: int) -> int:
    """Per-rank bytes of one MoE layer under tensor parallelism (NVFP4 experts, bf16 attention)."""
    H, I, E = cfg.hidden_size, cfg.moe_intermediate_size, cfg.n_routed_experts
    nv = lambda n: n * 9 // 16
    experts = nv((E + 1) * 3 * I * H) // world
    attn = 2 * (cfg.q_lora_rank * H + (cfg.kv_lora_rank + cfg.qk_rope_head_dim + cfg.index_head_dim + cfg.index_n_heads) * H
                + cfg.index_n_heads * cfg.index_head_dim * cfg.q_lora_rank
                + (cfg.num_attention_heads * (cfg.qk_head_dim) * cfg.q_lora_rank
                   + cfg.num_attention_heads * (cfg.qk_nope_head_dim + cfg.v_head_dim) * cfg.kv_lora_rank) // world)
    o = nv(cfg.num_attention_heads * cfg.v_head_dim * H) // world
    return experts + attn + o + 2 * E * H


def main():
    args = parse()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "reference is a Node.js/N-API addon compiled only for sm_120a "
                          "with an empty vendor/flashinfer submodule; `pip install` of the reference tree fails: no setup.py/pyproject.toml"}))
        return 0

    # the contract is ONE line on stdout: libraries that print there (NCCL's version banner) are sent to stderr for the
    # whole run, the JSON line goes to the saved descriptor at the end
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)

    import torch
    import torch.distributed as dist
    from slopllm_b200.config import GlmMoeDsaConfig
    from slopllm_b200.models.glm_moe_dsa import GlmMoeDsaModel
    from slopllm_b200.models.weights import random_model
    from slopllm_b200.parallel.dist import ParallelContext, init_from_env
    from slopllm_b200.parallel.fused import make_comm
    from slopllm_b200.runtime.engine import Engine
    from slopllm_b200.ops import native as N
    from slopllm_b200.ops import tcgen05

    ctx = init_from_env()
    W, rank, dev = ctx.world, ctx.rank, ctx.device
    assert dev.type == "cuda", "bench.py needs a GPU"
    torch.manual_seed(0)
    B, P, K, Wu = args.batch, args.prompt_len, args.steps, args.warmup

    def sync_barrier():
        torch.cuda.synchronize()
        if W > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if W == 1:
            return ms
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def ranks_agree(tokens) -> bool:
        """True when every rank holds the same token list (the tensor-parallel ranks of one replica must sample alike)."""
        if W == 1:
            return True
        t = torch.tensor([int(x) for x in tokens], dtype=torch.int64, device=dev)
        lo, hi = t.clone(), t.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        return bool((lo == hi).all().item())

    def pick_layers() -> int:
        if args.tiny:
            return args.layers or 4
        if args.layers:
            return args.layers
        if W == 1:
            return FIXED_LAYERS
        probe = GlmMoeDsaConfig.glm5(78)
        free, _ = torch.cuda.mem_get_info()
        fixed = 2 * probe.vocab_size * probe.hidden_size * (1 + 1 / W) + 14e9      # embed + lm_head shard + KV/workspace
        fit = int((free - fixed) // layer_bytes(probe, W)) - 1                     # one more for the MTP layer
        return max(4, min(78, fit))

    class Rig:
        """One model + engine; `close()` drops its graphs, buffers and peer mappings before the next one is built."""

        def __init__(self, layers: int, context: ParallelContext, pages_for_len: int, batch: int, mtp: int, weights=None):
            self.cfg = GlmMoeDsaConfig.glm5(num_layers=layers)
            t0 = time.time()
            self.weights = weights or random_model(self.cfg, 0, dev, torch.bfloat16, rank, W, exact=False, with_mtp=args.mtp > 0)
            torch.cuda.synchronize()
            self.t_init = time.time() - t0
            self.comm = make_comm(context, self.cfg, fused=not args.no_fused)
            self.model = GlmMoeDsaModel(self.cfg, self.weights, context, comm=self.comm)
            tokens_per_page = 64 * context.cp_world
            pages = (batch + 1) * (-(-pages_for_len // tokens_per_page) + 1)
            self.eng = Engine(self.cfg, self.model, pages, max_batch=batch, max_seq_len=pages_for_len, mtp=mtp)

        def check(self):
            tcgen05.check_errors(dev)
            self.eng.check_device_errors()

        def close(self, keep_weights: bool = False):
            sync_barrier()
            self.eng.graphs.entries.clear()
            if hasattr(self.comm, "close"):
                self.comm.close()
            w = self.weights if keep_weights else None
            self.eng = self.model = self.comm = self.weights = None
            gc.collect()
            torch.cuda.empty_cache()
            sync_barrier()
            return w

    def timed_decode(eng, seq_group, last_tokens, label):
        """K timed `decode_step` calls through the public API (e2e), then K device-timed
        graph replays of the same step."""
        cur = list(last_tokens)
        for _ in range(Wu):
            cur = eng.decode_step(seq_group, cur)
        h0, d0 = eng.h2d_bytes, eng.d2h_bytes
        sync_barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(K):
            cur = eng.decode_step(seq_group, cur)
        b.record()
        sync_barrier()
        e2e_ms = max_over_ranks(a.elapsed_time(b)) / K
        h2d, d2h = (eng.h2d_bytes - h0) // K, (eng.d2h_bytes - d0) // K
        agree = ranks_agree(cur)
        # device-only: replay the captured graph K times (inputs stay as last uploaded)
        key = next(k for k in eng.graphs.entries if k[0] == "decode" and k[1] == len(seq_group)
                   and eng.graphs.entries[k].graph is not None)
        gr = eng.graphs.entries[key]
        for _ in range(Wu):
            gr.graph.replay()
        sync_barrier()
        a.record()
        for _ in range(K):
            gr.graph.replay()
        b.record()
        sync_barrier()
        dev_ms = max_over_ranks(a.elapsed_time(b)) / K
        return {"label": label, "ms_per_step": dev_ms, "e2e_ms_per_step": e2e_ms, "h2d": h2d, "d2h": d2h,
                "launches_per_step": gr.launches, "kernels_per_step": getattr(gr, "kernels", gr.launches), "last": cur,
                "ranks_agree": agree}

    def decode_rig(layers: int, weights=None):
        total_steps = 4 * (K + Wu) + 64
        max_len = P + total_steps * (args.mtp + 1) + 64
        rig = Rig(layers, ctx, max_len, B, args.mtp, weights)
        g = torch.Generator().manual_seed(1)
        prompts = [torch.randint(0, rig.cfg.vocab_size, (P,), generator=g).tolist() for _ in range(B)]
        seqs = [rig.eng.kv.new_sequence() for _ in range(B)]
        sync_barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        last, _ = rig.eng.prefill(seqs, prompts, chunk_size=min(P, 4096), want_hidden=True)
        e1.record()
        sync_barrier()
        return rig, seqs, last, max_over_ranks(e0.elapsed_time(e1))

    # =================================== headline: decode, batch 8, MTP off ===================================
    L = pick_layers()
    rig, seqs, last, prefill_ms = decode_rig(L)
    cfg, eng = rig.cfg, rig.eng
    sampler = ClockSampler(dev.index or 0)
    if rank == 0:
        sampler.start()
    r8 = timed_decode(eng, seqs, last, f"bs{B}")
    clocks = sampler.stop() if rank == 0 else {}

    details = {"prefill_tok_s": B * P / (prefill_ms / 1e3), "prefill_ms": prefill_ms, "weights_init_s": rig.t_init,
               "weights_gb_per_rank": rig.weights.nbytes() / 1e9, "ranks_sample_alike": r8["ranks_agree"]}
    if not args.skip_details:
        # the side measurements must not cost the headline line: a failure here is recorded, not raised
        try:
            r1 = timed_decode(eng, seqs[:1], r8["last"][:1], "bs1")
            details["bs1"] = {"tok_s": 1e3 / r1["ms_per_step"], "ms_per_step": r1["ms_per_step"],
                              "ms_per_layer": r1["ms_per_step"] / L, "e2e_tok_s": 1e3 / r1["e2e_ms_per_step"],
                              "launches_per_step": r1["launches_per_step"], "ranks_sample_alike": r1["ranks_agree"]}
            if args.mtp > 0:
                for grp, name, ref in ((seqs[:1], "bs1", BASELINE_BS1_STEPS_S), (seqs, f"bs{B}", BASELINE_BS8_STEPS_S)):
                    lt = r1["last"] if name == "bs1" else r8["last"]
                    hs = [torch.zeros(1, cfg.hidden_size, dtype=torch.bfloat16, device=dev) for _ in grp]
                    seed = eng.mtp_seed(grp, lt, hs)
                    acc_tokens = 0
                    for _ in range(Wu):
                        _, lt, seed = eng.mtp_decode_step(grp, lt, seed)
                    sync_barrier()
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record()
                    for _ in range(K):
                        acc, lt, seed = eng.mtp_decode_step(grp, lt, seed)
                        acc_tokens += sum(len(x) for x in acc)
                    b.record()
                    sync_barrier()
                    ms = max_over_ranks(a.elapsed_time(b)) / K
                    details[f"mtp{args.mtp}_{name}"] = {
                        "steps_s": 1e3 / ms, "ms_per_step": ms, "tok_s": acc_tokens / (ms * K / 1e3),
                        "accept_len": acc_tokens / (K * len(grp)),
                        # the reference's figure is tok/s divided by the accept length, i.e. sequence-steps per second
                        "seq_steps_s": len(grp) * 1e3 / ms,
                        "vs_ref_steps_s": (len(grp) * 1e3 / ms) / ref if L == 78 else None,
                        "ranks_sample_alike": ranks_agree(lt),
                        "note": "random-init weights: drafts are almost never accepted, so tok/s ~= steps/s * batch"}
        except Exception as err:  # noqa: BLE001
            details["error"] = f"{type(err).__name__}: {err}"
    rig.check()
    weights = rig.close(keep_weights=True)
    eng = None

    # =================================== like-for-like: the one-GPU layer count at every N ===================================
    if not args.skip_fixed and not args.tiny and L != FIXED_LAYERS:
        try:
            weights = None
            gc.collect()
            torch.cuda.empty_cache()
            rig_f, seqs_f, last_f, _ = decode_rig(FIXED_LAYERS)
            rf = timed_decode(rig_f.eng, seqs_f, last_f, f"bs{B}")
            details["fixed_layers"] = {"layers": FIXED_LAYERS, "ms_per_step": rf["ms_per_step"], "tok_s": B * 1e3 / rf["ms_per_step"],
                                       "ms_per_layer": rf["ms_per_step"] / FIXED_LAYERS, "ranks_sample_alike": rf["ranks_agree"]}
            rig_f.check()
            rig_f.close()
            rig_f = None
        except Exception as err:  # noqa: BLE001
            details["fixed_layers"] = {"error": f"{type(err).__name__}: {err}"}
    elif L == FIXED_LAYERS:
        details["fixed_layers"] = {"layers": L, "ms_per_step": r8["ms_per_step"], "tok_s": B * 1e3 / r8["ms_per_step"],
                                   "ms_per_layer": r8["ms_per_step"] / L, "note": "same run as the headline"}

    # =================================== serving: 8 requests, shared prefix, MTP 3 (full model only) ===================================
    full_model = L == 78 or args.tiny
    if args.skip_serving or not full_model:
        details["batch8_prefix"] = None if args.skip_serving else {"skipped": f"needs the full 78-layer model ({L} layers fit on {W} GPU(s))"}
    else:
        try:
            details["batch8_prefix"] = serving_run(args, ctx, dev, L, weights, sync_barrier, max_over_ranks, ranks_agree, Rig)
        except Exception as err:  # noqa: BLE001
            details["batch8_prefix"] = {"error": f"{type(err).__name__}: {err}"}

    # =================================== 128K prefill under context parallelism (full model, 8 GPUs) ===================================
    if args.skip_cp or not full_model or (W < 4 and not (args.tiny and W > 1)):
        details["prefill_128k_cp"] = None if args.skip_cp else {"skipped": f"needs the full model on 4 or 8 GPUs (have {L} layers on {W})"}
    else:
        try:
            details["prefill_128k_cp"] = cp_run(args, ctx, dev, L, weights, sync_barrier, max_over_ranks, Rig)
        except Exception as err:  # noqa: BLE001
            details["prefill_128k_cp"] = {"error": f"{type(err).__name__}: {err}"}

    tok_s = B * 1e3 / r8["ms_per_step"]
    out = {
        "metric": f"decode_tok_s_bs{B}", "value": tok_s, "unit": "tokens/s", "n_gpus": W, "steps": K, "warmup": Wu,
        "ms_per_step": r8["ms_per_step"], "ms_per_layer": r8["ms_per_step"] / L, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16 activations, NVFP4/bf16 weights",
        "data": "synthetic token ids, random-init NVFP4 weights",
        "config": {"model": "GLM-5-class glm_moe_dsa NVFP4", "layers": L, "layers_full_model": 78,
                   "global_batch": B, "seq_len": P, "parallelism": f"tp{W}", "mtp": 0,
                   "l2": "inputs larger than L2: every step streams the active weights (GBs per rank) from HBM",
                   "baseline_note": "the reference publishes no MTP-off throughput, so vs_baseline is null; the comparable figures "
                                    "are details.mtp3_*.vs_ref_steps_s (sequence-steps/s against the reference's MTP-normalised "
                                    "60.8 / 163.5 on 8x RTX PRO 6000) and details.prefill_128k_cp.vs_ref"},
        "clocks": clocks,
        "e2e": {"value": B * 1e3 / r8["e2e_ms_per_step"], "unit": "tokens/s", "h2d_bytes_per_step": r8["h2d"],
                "d2h_bytes_per_step": r8["d2h"]},
        "gpu_launches": r8["kernels_per_step"] * K,
        "details": details,
    }
    if rank == 0:
        sys.stdout.flush()
        os.write(real_stdout, (json.dumps(out) + "\n").encode())
    sync_barrier()
    weights = None
    gc.collect()
    if W > 1:
        dist.destroy_process_group()
    return 0


def serving_run(args, ctx, dev, L, weights, sync_barrier, max_over_ranks, ranks_agree, Rig):
    """8 requests of 8192 prompt tokens whose first 4096 are common, through the continuous-batching scheduler with a chunk
    budget of 8192 tokens and MTP drafts; every rank runs the same scheduler on the same requests (no front end)."""
    import torch
    from slopllm_b200.config import SamplingParams
    from slopllm_b200.scheduler.scheduler import GenerationRequest, GenerationScheduler
    n_req, plen, shared, dec = 8, 8192, 4096, args.serving_decode
    if args.tiny:
        plen, shared, dec = 512, 256, min(dec, 32)
    rig = Rig(L, ctx, plen + dec + 4 * (args.mtp + 1) + 64, n_req, args.mtp, weights)
    sched = GenerationScheduler(rig.eng, max_batch=n_req, chunk_size=8192, eos_token_ids=())
    g = torch.Generator().manual_seed(7)
    common = torch.randint(0, rig.cfg.vocab_size, (shared,), generator=g).tolist()
    reqs = [GenerationRequest(id=f"r{i}", input_ids=common + torch.randint(0, rig.cfg.vocab_size, (plen - shared,), generator=g).tolist(),
                              max_tokens=dec, sampling=SamplingParams(temperature=0.0)) for i in range(n_req)]
    sync_barrier()
    t0 = time.time()
    # the first request arrives alone; the others follow once its prompt is cached, so that they find the common prefix
    reqs[0].submitted_at = time.time()
    sched.submit(reqs[0])
    while reqs[0].first_token_at is None and not reqs[0].finish_reason:
        sched.step()
    for r in reqs[1:]:
        r.submitted_at = time.time()
        sched.submit(r)
    while not all(r.finish_reason for r in reqs):
        sched.step()
    torch.cuda.synchronize()
    t_all = time.time() - t0
    errs = [r.error for r in reqs if r.error]
    ttft = sorted((r.first_token_at - r.submitted_at) for r in reqs if r.first_token_at)
    t_first_decode = max(r.first_token_at for r in reqs if r.first_token_at)
    gen = sum(len(r.generated) for r in reqs)
    decode_s = max_over_ranks((t0 + t_all - t_first_decode) * 1e3) / 1e3
    out = {"requests": n_req, "prompt_tokens": plen, "shared_prefix": shared, "decode_tokens_per_request": dec, "mtp": args.mtp,
           "cached_prompt_tokens": sum(r.cached_tokens for r in reqs),
           "p50_ttft_s": statistics.median(ttft) if ttft else None, "ttft_s": [round(x, 3) for x in ttft],
           "generated_tokens": gen, "total_s": max_over_ranks(t_all * 1e3) / 1e3,
           "decode_tok_s": gen / max(decode_s, 1e-9),
           "note": "decode_tok_s: tokens generated after the last request's first token / that time (all 8 rows decoding); "
                   "host clock around the scheduler loop",
           "ranks_sample_alike": ranks_agree([t for r in reqs for t in r.generated[:4]]), "errors": errs[:2]}
    rig.check()
    rig.close(keep_weights=True)
    return out


def cp_run(args, ctx, dev, L, weights, sync_barrier, max_over_ranks, Rig):
    """One long prompt prefilled in 8192-token chunks with the KV tokens interleaved over the ranks, then 128 decode steps."""
    import torch
    from slopllm_b200.parallel.dist import ParallelContext
    n, n_dec = args.cp_context, 128
    cctx = ParallelContext(ctx.rank, ctx.world, ctx.device, True, ctx.ep, ctx.group)
    rig = Rig(L, cctx, n + n_dec + 64, 1, 0, weights)
    eng = rig.eng
    g = torch.Generator().manual_seed(11)
    prompt = torch.randint(0, rig.cfg.vocab_size, (n,), generator=g).tolist()
    s = eng.kv.new_sequence()
    sync_barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    last, _ = eng.prefill([s], [prompt], chunk_size=8192)
    b.record()
    sync_barrier()
    ms = max_over_ranks(a.elapsed_time(b))
    cur = [last[0]]
    for _ in range(4):
        cur = eng.decode_step([s], cur)
    sync_barrier()
    a.record()
    for _ in range(n_dec):
        cur = eng.decode_step([s], cur)
    b.record()
    sync_barrier()
    dms = max_over_ranks(a.elapsed_time(b)) / n_dec
    out = {"context": n, "chunk": 8192, "cp": ctx.world, "prefill_s": ms / 1e3, "prefill_tok_s": n / (ms / 1e3),
           "vs_ref": (n / (ms / 1e3)) / BASELINE_PREFILL_128K_TOK_S if n == 131072 else None,
           "decode_ms_per_token": dms, "decode_tokens": n_dec}
    rig.check()
    rig.close()
    return out


if __name__ == "__main__":
    sys.exit(main())
