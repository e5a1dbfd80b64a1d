"""Plumbing model (tiny glm_moe_dsa, fp32 dequantised NVFP4) on CPU ranks over gloo:
TP=2, CP=2 and EP=2 must reproduce the single-rank greedy tokens.
Mirrors the reference's TP=1 vs TP=2 / CP on-off model tests (`tests/test_glm51.ts`)."""
import torch

from slopllm_b200.config import GlmMoeDsaConfig
from slopllm_b200.models.glm_moe_dsa import GlmMoeDsaModel, KVCacheTensors, make_step
from slopllm_b200.models.weights import random_model
from slopllm_b200.parallel.dist import ParallelContext, init_from_env

from mp_util import run_ranks

PROMPT, NEW = 128, 32


def _greedy(rank, world, cp, ep, prompt_len, new):
    ctx = init_from_env("gloo", cp=cp, ep=ep) if world > 1 else ParallelContext()
    cfg = GlmMoeDsaConfig.tiny()
    w = random_model(cfg, 0, tp_rank=ctx.rank, tp_world=ctx.world, ep=ep)
    m = GlmMoeDsaModel(cfg, w, ctx)
    cache = KVCacheTensors.allocate(cfg, 8, "cpu")
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab_size, (prompt_len,), generator=g).tolist()
    pt = [[0, 1, 2, 3, 4, 5, 6, 7]]
    st = make_step(prompt, list(range(prompt_len)), [0] * prompt_len, pt, ctx, logits_idx=[prompt_len - 1])
    toks = [int(m.forward(st, cache).argmax(-1))]
    for i in range(new - 1):
        st = make_step([toks[-1]], [prompt_len + i], [0], pt, ctx)
        toks.append(int(m.forward(st, cache).argmax(-1)))
    return toks


def test_single_rank_deterministic():
    a = _greedy(0, 1, False, False, PROMPT, 8)
    b = _greedy(0, 1, False, False, PROMPT, 8)
    assert a == b and len(set(a)) > 1


def test_tp2_matches_tp1():
    ref = _greedy(0, 1, False, False, PROMPT, NEW)
    out = run_ranks(_greedy, 2, False, False, PROMPT, NEW)
    assert out[0] == out[1] == ref


def test_cp2_matches_single():
    ref = _greedy(0, 1, False, False, PROMPT, 12)
    out = run_ranks(_greedy, 2, True, False, PROMPT, 12)
    assert out[0] == out[1] == ref


def _greedy_gather(rank, world, prompt_len, new):
    import os
    os.environ["SLOPLLM_B200_CP_GATHER_KV"] = "1"
    return _greedy(rank, world, True, False, prompt_len, new)


def test_cp2_gather_kv_mode_matches_single():
    """Fallback CP mode: KV stays sharded by token, every layer's rows are gathered into a flat replicated
    buffer and each rank attends like a TP rank (no top-k or partial merge)."""
    ref = _greedy(0, 1, False, False, PROMPT, 10)
    out = run_ranks(_greedy_gather, 2, PROMPT, 10)
    assert out[0] == out[1] == ref


def test_ep2_matches_single():
    """Expert parallelism as masked partial sums (the default: no dispatch, every rank runs its own experts on the replicated
    rows and the following all-reduce adds the ranks up)."""
    ref = _greedy(0, 1, False, False, 40, 6)
    out = run_ranks(_greedy, 2, False, True, 40, 6)
    assert out[0] == out[1] == ref


def _greedy_a2a(rank, world, prompt_len, new):
    import slopllm_b200.models.glm_moe_dsa as M
    M.EP_ALL_TO_ALL = True                      # token-split dispatch / combine all-to-all
    return _greedy(rank, world, False, True, prompt_len, new)


def test_ep2_all_to_all_variant_matches_single():
    ref = _greedy(0, 1, False, False, 40, 6)
    out = run_ranks(_greedy_a2a, 2, 40, 6)
    assert out[0] == out[1] == ref


def _gather_many(rank, world):
    import torch
    from slopllm_b200.parallel.dist import Comm, init_from_env
    comm = Comm(init_from_env("gloo"))
    a = torch.full((3, 2, 5), float(rank + 1), dtype=torch.bfloat16)        # 60 bytes: segment padded to 64
    b = torch.arange(7, dtype=torch.float32).reshape(1, 7) + 10 * rank       # 28 bytes
    c = torch.tensor([[rank, -rank]], dtype=torch.int32)
    ga, gb, gc = comm.all_gather_many([a, b, c], dim=1)
    one = comm.all_gather(a, dim=1)
    return ga.shape, bool(torch.equal(ga, one)), gb.tolist(), gc.tolist()


def test_all_gather_many_packs_several_tensors_into_one_collective():
    from mp_util import run_ranks
    for shape, same, gb, gc in run_ranks(_gather_many, 2):
        assert tuple(shape) == (3, 4, 5) and same
        assert gb == [[0, 1, 2, 3, 4, 5, 6, 10, 11, 12, 13, 14, 15, 16]]
        assert gc == [[0, 0, 1, -1]]
