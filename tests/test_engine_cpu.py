"""Engine logic on the CPU reference op set: chunked prefill == whole prefill, MTP
speculative decode (greedy verification) == plain greedy decode, page bookkeeping."""
import torch

from slopllm_b200.config import GlmMoeDsaConfig
from slopllm_b200.models.glm_moe_dsa import GlmMoeDsaModel
from slopllm_b200.models.weights import random_model
from slopllm_b200.runtime.engine import Engine


def _engine(cfg, w, mtp=0, pages=16):
    return Engine(cfg, GlmMoeDsaModel(cfg, w), num_pages=pages, max_batch=2, max_seq_len=512, cuda_graph=False, mtp=mtp)


def test_chunked_prefill_and_mtp_equal_plain_greedy():
    cfg = GlmMoeDsaConfig.tiny()
    w = random_model(cfg, 0)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg.vocab_size, (90,), generator=g).tolist() for _ in range(2)]

    def plain(chunk):
        eng = _engine(cfg, w)
        seqs = [eng.kv.new_sequence() for _ in range(2)]
        last, _ = eng.prefill(seqs, prompts, chunk_size=chunk)
        toks = [[t] for t in last]
        for _ in range(8):
            last = eng.decode_step(seqs, last)
            for b in range(2):
                toks[b].append(last[b])
        return toks

    a, b = plain(512), plain(32)
    assert a == b

    eng = _engine(cfg, w, mtp=3)
    seqs = [eng.kv.new_sequence() for _ in range(2)]
    last, hid = eng.prefill(seqs, prompts, chunk_size=64, want_hidden=True)
    seed = eng.mtp_seed(seqs, last, hid)
    streams = [[t] for t in last]
    steps = 0
    while min(len(s) for s in streams) < 9:
        acc, last, seed = eng.mtp_decode_step(seqs, last, seed)
        steps += 1
        for i in range(2):
            assert 1 <= len(acc[i]) <= 4
            streams[i] += acc[i]
    assert [s[:9] for s in streams] == a
    for s in seqs:
        assert len(s.pages) == eng.kv.pages_for(s.length)


def test_phased_prefill_matches_plain_prefill():
    """Two half-chunks walking the layers in lock step give the same next token and hidden state as one chunk."""
    import torch
    from slopllm_b200.config import GlmMoeDsaConfig
    from slopllm_b200.models.glm_moe_dsa import GlmMoeDsaModel
    from slopllm_b200.models.weights import random_model
    from slopllm_b200.runtime.engine import Engine
    cfg = GlmMoeDsaConfig.tiny()
    w = random_model(cfg, 0)
    prompt = torch.randint(0, cfg.vocab_size, (300,), generator=torch.Generator().manual_seed(3)).tolist()
    outs = []
    for phased in (False, True):
        eng = Engine(cfg, GlmMoeDsaModel(cfg, w), num_pages=16, max_batch=1, max_seq_len=512, cuda_graph=False,
                     phased_prefill=phased, phased_min_tokens=128)
        s = eng.kv.new_sequence()
        tok, hid = eng.prefill([s], [prompt], chunk_size=256, want_hidden=True)      # chunk 1 phased (256), chunk 2 plain (44)
        nxt = eng.decode_step([s], tok)
        outs.append((tok, nxt, hid[0]))
    assert outs[0][0] == outs[1][0] and outs[0][1] == outs[1][1]
    assert torch.allclose(outs[0][2], outs[1][2], atol=1e-4, rtol=1e-4)


def test_host_tier_restores_pages_of_the_real_engine():
    """Pinned-host prefix tier with the real engine's page IO: a finished conversation is evicted to the host, the GPU tier
    is flushed, and the same prompt comes back with its prefix restored from host pages and the same greedy tokens."""
    import torch
    from slopllm_b200.config import GlmMoeDsaConfig, SamplingParams
    from slopllm_b200.models.glm_moe_dsa import GlmMoeDsaModel
    from slopllm_b200.models.weights import random_model
    from slopllm_b200.runtime.engine import Engine
    from slopllm_b200.scheduler.scheduler import GenerationRequest, GenerationScheduler, HostTier
    cfg = GlmMoeDsaConfig.tiny()
    eng = Engine(cfg, GlmMoeDsaModel(cfg, random_model(cfg, 0)), num_pages=8, max_batch=1, max_seq_len=512, cuda_graph=False)
    assert eng.supports_host_tier()
    # page IO round trip: every layer's rows of the page, and nothing else, come back
    for lc in eng.cache.layers:
        lc.kv.random_(0, 255)
        if lc.idx is not None:
            lc.idx.random_(0, 255)
    want = [(lc.kv[64:128].clone(), None if lc.idx is None else lc.idx[64:128].clone()) for lc in eng.cache.layers]
    blob = eng.read_page(1)
    assert blob.dtype == torch.uint8 and blob.numel() == sum(64 * (lc.kv.shape[1] + (lc.idx.shape[1] if lc.idx is not None else 0))
                                                            for lc in eng.cache.layers)
    eng.write_page(5, blob)
    for lc, (kv, idx) in zip(eng.cache.layers, want):
        assert torch.equal(lc.kv[320:384], kv) and (idx is None or torch.equal(lc.idx[320:384], idx))
        assert torch.equal(lc.kv[64:128], kv)
    import pytest
    with pytest.raises(ValueError):
        eng.write_page(5, blob[:-16])
    # batched form: several pages in one gather / one copy, same bytes as page by page
    blobs = eng.read_pages([1, 5, 2])
    assert torch.equal(blobs[0], blob) and torch.equal(blobs[1], eng.read_page(5)) and torch.equal(blobs[2], eng.read_page(2))
    eng.write_pages([6, 7], [blobs[2], blobs[0]])
    assert torch.equal(eng.read_page(6), blobs[2]) and torch.equal(eng.read_page(7), blob)
    with pytest.raises(ValueError):
        eng.write_pages([6], [blob[:-16]])
    # scheduler level
    tier = HostTier(8, eng.kv.tokens_per_page, eng.read_page, eng.write_page, read_pages=eng.read_pages, write_pages=eng.write_pages)
    sched = GenerationScheduler(eng, max_batch=1, chunk_size=256, host_tier=tier)
    prompt = torch.randint(2, cfg.vocab_size, (150,), generator=torch.Generator().manual_seed(11)).tolist()

    def run(i):
        r = GenerationRequest(id=str(i), input_ids=list(prompt), max_tokens=4, sampling=SamplingParams(temperature=0.0))
        sched.submit(r)
        for _ in range(100):
            sched.step()
            if r.finish_reason:
                sched.step()
                return r
        raise AssertionError("request did not finish")
    first = run(0)
    assert first.cached_tokens == 0 and len(first.generated) == 4
    ev = sched.flush_gpu_cache()                   # staged pages go to the host tier, the GPU tier is emptied
    sched.step()
    assert ev.done.is_set() and tier.used_pages == 2 and not eng.kv.staged
    for lc in eng.cache.layers:                    # whatever the GPU pages held is gone
        lc.kv.zero_()
        if lc.idx is not None:
            lc.idx.zero_()
    again = run(1)
    assert again.cached_tokens == 128              # two pages restored from the host
    assert again.generated == first.generated


def test_dense_cache_page_io_and_hybrid_refusal():
    import torch
    from slopllm_b200.models.dense import DenseConfig, DenseModel, random_dense_model
    from slopllm_b200.runtime.engine import Engine
    cfg = DenseConfig.tiny()
    w, _ = random_dense_model(cfg, seed=1, device="cpu", dtype=torch.float32)
    eng = Engine(cfg, DenseModel(cfg, w), num_pages=4, max_batch=1, max_seq_len=256, cuda_graph=False)
    assert eng.supports_host_tier()
    for t in eng.cache.page_tensors():
        t.normal_()
    blob = eng.read_page(2)
    eng.write_page(0, blob)
    for t in eng.cache.page_tensors():
        assert torch.equal(t[0:64], t[128:192])
    hyb = DenseConfig.tiny(hybrid=True)
    wh, _ = random_dense_model(hyb, seed=1, device="cpu", dtype=torch.float32)
    assert not Engine(hyb, DenseModel(hyb, wh), num_pages=4, max_batch=1, max_seq_len=256, cuda_graph=False).supports_host_tier()
