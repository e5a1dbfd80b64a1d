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
