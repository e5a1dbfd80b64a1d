"""Qwen3 / Qwen3.5 families: the paged engine against a straightforward full-sequence fp32
implementation of the same architecture (HF semantics) built from the same checkpoint tensors.

Mirrors the reference's model-level tests (`tests/python/qwen3_model.py`, `qwen35_model.py`
as oracles of the TypeScript models).
"""
import pytest
import torch

from slopllm_b200.models.dense import DenseConfig, DenseModel, random_dense_model
from slopllm_b200.ops import reference as R
from slopllm_b200.parallel.dist import ParallelContext
from slopllm_b200.runtime.engine import Engine


def oracle_logits(cfg: DenseConfig, t: dict, ids: torch.Tensor) -> torch.Tensor:
    """Whole-sequence forward in fp32, no cache: logits [T, V]."""
    pfx = cfg.weight_prefix
    f = lambda n: t[n].to(torch.float32)
    nw = lambda n: f(n) + (1.0 if cfg.gemma_norm else 0.0)
    T = ids.shape[0]
    pos = torch.arange(T)
    x = f(pfx + "embed_tokens.weight")[ids]
    hd = cfg.head_dim
    for i, kind in enumerate(cfg.layer_types):
        lp = f"{pfx}layers.{i}."
        h = R.rmsnorm(x, nw(lp + "input_layernorm.weight"), cfg.rms_norm_eps)
        if kind == "full_attention":
            qs = hd * (2 if cfg.attn_output_gate else 1)
            qg = (h @ f(lp + "self_attn.q_proj.weight").t()).view(T, cfg.num_attention_heads, qs)
            q, gate = qg[..., :hd], qg[..., hd:]
            k = (h @ f(lp + "self_attn.k_proj.weight").t()).view(T, cfg.num_key_value_heads, hd)
            v = (h @ f(lp + "self_attn.v_proj.weight").t()).view(T, cfg.num_key_value_heads, hd)
            q = R.rmsnorm(q, nw(lp + "self_attn.q_norm.weight"), cfg.rms_norm_eps)
            k = R.rmsnorm(k, nw(lp + "self_attn.k_norm.weight"), cfg.rms_norm_eps)
            q = R.apply_rope(q, pos, cfg.rope_theta, cfg.rope_dim, interleave=False)
            k = R.apply_rope(k, pos, cfg.rope_theta, cfg.rope_dim, interleave=False)
            o = R.dense_attention(q, k, v, cfg.scaling)
            if cfg.attn_output_gate:
                o = o * torch.sigmoid(gate)
            a = o.reshape(T, -1) @ f(lp + "self_attn.o_proj.weight").t()
        else:
            lh, dk, dv = cfg.linear_num_key_heads, cfg.linear_key_head_dim, cfg.linear_value_head_dim
            qkv = h @ f(lp + "linear_attn.in_proj_qkv.weight").t()
            z = (h @ f(lp + "linear_attn.in_proj_z.weight").t()).view(T * lh, dv)
            av = h @ f(lp + "linear_attn.in_proj_a.weight").t()
            bv = h @ f(lp + "linear_attn.in_proj_b.weight").t()
            conv, _ = R.causal_conv1d(qkv, f(lp + "linear_attn.conv1d.weight").reshape(cfg.conv_dim, -1), None, None, True)
            q = conv[:, :lh * dk].view(T, lh, dk)
            k = conv[:, lh * dk:2 * lh * dk].view(T, lh, dk)
            v = conv[:, 2 * lh * dk:].view(T, lh, dv)
            q = q * torch.rsqrt((q * q).sum(-1, keepdim=True) + 1e-8) * dk ** -0.5
            k = k * torch.rsqrt((k * k).sum(-1, keepdim=True) + 1e-8)
            g = -torch.exp(f(lp + "linear_attn.A_log")) * torch.nn.functional.softplus(av + f(lp + "linear_attn.dt_bias"))
            o, _ = R.gdn_recurrent(q, k, v, g, torch.sigmoid(bv), torch.zeros(lh, dk, dv))
            o = R.rmsnorm_gated(o.reshape(T * lh, dv), z, f(lp + "linear_attn.norm.weight"), cfg.rms_norm_eps)
            a = o.reshape(T, lh * dv) @ f(lp + "linear_attn.out_proj.weight").t()
        x = x + a
        h = R.rmsnorm(x, nw(lp + "post_attention_layernorm.weight"), cfg.rms_norm_eps)
        gate_up = torch.nn.functional.silu(h @ f(lp + "mlp.gate_proj.weight").t()) * (h @ f(lp + "mlp.up_proj.weight").t())
        x = x + gate_up @ f(lp + "mlp.down_proj.weight").t()
    x = R.rmsnorm(x, nw(pfx + "norm.weight"), cfg.rms_norm_eps)
    head = t.get("lm_head.weight", t[pfx + "embed_tokens.weight"])
    return x @ head.to(torch.float32).t()


def run_engine(cfg, w, device, prompt, n_new, chunk):
    ctx = ParallelContext(device=torch.device(device))
    model = DenseModel(cfg, w, ctx)
    eng = Engine(cfg, model, num_pages=16, max_batch=2, max_seq_len=512, cuda_graph=False)
    s, cached = eng.kv.start_request(prompt)
    assert cached == 0
    toks, _ = eng.prefill([s], [prompt], chunk_size=chunk)
    out = [toks[0]]
    for _ in range(n_new - 1):
        out.append(eng.decode_step([s], [out[-1]])[0])
    return out


def teacher_forced_errors(cfg, w, tensors, device, prompt, steps, chunk):
    """Chunked prefill then `steps` decode steps fed with the oracle's tokens; returns the largest logits
    error relative to the logits' peak at each step."""
    ctx = ParallelContext(device=torch.device(device))
    model = DenseModel(cfg, w, ctx)
    eng = Engine(cfg, model, num_pages=16, max_batch=2, max_seq_len=512, cuda_graph=False)
    s, cached = eng.kv.start_request(prompt)
    assert cached == 0
    _, hid = eng.prefill([s], [prompt], chunk_size=chunk, want_hidden=True)
    h = hid[0]
    ids, errs = list(prompt), []
    for _ in range(steps):
        want = oracle_logits(cfg, tensors, torch.tensor(ids))[-1]
        got = model.compute_logits(h)[-1].to(torch.float32).cpu()
        errs.append(((want - got).abs().max() / want.abs().max()).item())
        nxt = int(want.argmax())
        pos = s.length
        eng.kv.append_tokens(s, [nxt])
        st = eng._eager_state([nxt], [pos], [0], [s], max_kv_len=pos + 1)
        eng._prepare(st, [s])
        h = model.forward_hidden(st, eng.cache)
        eng.kv.report_tokens(s)
        ids.append(nxt)
    return errs


@pytest.mark.parametrize("hybrid", [False, True])
def test_dense_engine_matches_oracle_cpu(hybrid):
    cfg = DenseConfig.tiny(hybrid=hybrid)
    w, tensors = random_dense_model(cfg, seed=3, device="cpu", dtype=torch.float32)
    prompt = torch.randint(2, cfg.vocab_size, (70,), generator=torch.Generator().manual_seed(5)).tolist()
    errs = teacher_forced_errors(cfg, w, tensors, "cpu", prompt, 5, chunk=32)      # 3 prefill chunks, then decode
    assert max(errs) < 2e-2, errs
    # free-running generation through the public engine calls works too
    assert len(run_engine(cfg, w, "cpu", prompt, 3, chunk=32)) == 3


def test_config_parsing_qwen35():
    raw = {"model_type": "qwen3_5", "text_config": {
        "hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 2, "num_attention_heads": 2, "num_key_value_heads": 1,
        "head_dim": 32, "vocab_size": 100, "layer_types": ["linear_attention", "full_attention"], "attn_output_gate": True,
        "rope_parameters": {"rope_theta": 5e5, "partial_rotary_factor": 0.25}, "linear_num_key_heads": 2,
        "linear_num_value_heads": 2, "linear_key_head_dim": 64, "linear_value_head_dim": 64}}
    cfg = DenseConfig.from_hf_dict(raw)
    assert cfg.model_type == "qwen3_5" and cfg.rope_dim == 8 and cfg.gemma_norm and cfg.weight_prefix == "model.language_model."
    assert cfg.layer_types == ["linear_attention", "full_attention"] and cfg.conv_dim == 2 * (128 + 64)


def test_fp8_block_roundtrip():
    from slopllm_b200.ops import dense as D
    w = torch.randn(200, 300, generator=torch.Generator().manual_seed(0))
    q, s = D.fp8_block_quantize(w)
    back = D.fp8_block_dequant(q, s).to(torch.float32)
    assert (back - w).abs().max() / w.abs().max() < 0.07


@pytest.mark.gpu
@pytest.mark.parametrize("hybrid", [False, True])
def test_dense_engine_gpu_matches_oracle(hybrid):
    """sm_100a kernels (paged GQA prefill / decode, norm+rope+cache write, GDN scan, conv1d, gated norm)
    inside the engine against the fp32 whole-sequence oracle."""
    cfg = DenseConfig.tiny(hybrid=hybrid)
    _, tensors = random_dense_model(cfg, seed=3, device="cpu", dtype=torch.float32)
    w_gpu, _ = random_dense_model(cfg, seed=3, device="cuda", dtype=torch.bfloat16)
    prompt = torch.randint(2, cfg.vocab_size, (150,), generator=torch.Generator().manual_seed(7)).tolist()
    errs = teacher_forced_errors(cfg, w_gpu, tensors, "cuda", prompt, 4, chunk=64)
    assert max(errs) < 6e-2, errs


def _fp8_checkpoint(cfg, seed=3):
    """Random checkpoint whose attention / MLP projections are FP8 block-quantised (`weight` + `weight_scale_inv`),
    and the same checkpoint with those projections expanded back to fp32 (what the oracle sees)."""
    from slopllm_b200.ops import dense as D
    _, tensors = random_dense_model(cfg, seed=seed, device="cpu", dtype=torch.float32)
    q8, plain = {}, {}
    for name, t in tensors.items():
        if name.endswith("_proj.weight") and "layers." in name and "linear_attn" not in name:
            q, s = D.fp8_block_quantize(t.to(torch.float32) * 8.0)          # spread the values over the e4m3 range
            q8[name], q8[name + "_scale_inv"] = q, s / 8.0
            plain[name] = D.fp8_block_dequant(q, s / 8.0).to(torch.float32)
        else:
            q8[name] = plain[name] = t
    return q8, plain


@pytest.mark.parametrize("world", [1, 2])
def test_fp8_weights_kept_match_expanded(world):
    """Keeping the FP8 projections in FP8 (sharded on scale-block edges, expanded where a shard edge cuts a block)
    gives the same weights as expanding them at load."""
    from slopllm_b200.models.dense import assemble_dense_weights
    cfg = DenseConfig.tiny()
    q8, _ = _fp8_checkpoint(cfg)
    kept_fp8 = 0
    for rank in range(world):
        a = assemble_dense_weights(cfg, q8, "cpu", torch.float32, rank, world, keep_fp8=True)
        b = assemble_dense_weights(cfg, q8, "cpu", torch.float32, rank, world, keep_fp8=False)
        for la, lb in zip(a.layers, b.layers):
            for f in ("w_qkv", "o_proj", "mlp_w13", "mlp_w2"):
                wa, wb = getattr(la, f), getattr(lb, f)
                assert not wb.is_fp8
                kept_fp8 += int(wa.is_fp8)
                # the expanded path rounds to bf16 once
                assert torch.equal(wa.dequant(torch.float32).to(torch.bfloat16), wb.weight.to(torch.bfloat16)), (rank, f)
    assert kept_fp8 > 0


def test_fp8_kept_engine_matches_oracle_cpu():
    from slopllm_b200.models.dense import assemble_dense_weights
    cfg = DenseConfig.tiny()
    q8, plain = _fp8_checkpoint(cfg)
    w = assemble_dense_weights(cfg, q8, "cpu", torch.float32, keep_fp8=True)
    assert w.layers[0].w_qkv.is_fp8 and w.layers[0].mlp_w2.is_fp8
    prompt = torch.randint(2, cfg.vocab_size, (40,), generator=torch.Generator().manual_seed(5)).tolist()
    errs = teacher_forced_errors(cfg, w, plain, "cpu", prompt, 2, chunk=32)
    assert max(errs) < 2e-2, errs


@pytest.mark.gpu
@pytest.mark.parametrize("T", [1, 2, 3, 8, 20, 100])
@pytest.mark.parametrize("out_f32", [False, True])
def test_fp8_linear_kernels(T, out_f32):
    """FP8 weight streaming (up to 8 rows) and the expand + GEMM path (more rows) against the fp32 definition."""
    from slopllm_b200.models.weights import LinearWeight
    from slopllm_b200.ops import dense as D
    from slopllm_b200.ops.cuda_ops import CudaOps
    g = torch.Generator().manual_seed(T)
    N_, K = 1300, 1408                   # neither a multiple of 128 x 8 nor of 512: ragged last scale blocks and K tail
    q, s = D.fp8_block_quantize(torch.randn(N_, K, generator=g))
    w = LinearWeight(q.cuda(), fp8_scale=s.cuda())
    x = torch.randn(T, K, generator=g).to(torch.bfloat16).cuda()
    ops = CudaOps(DenseConfig.tiny())
    y = ops.linear(x, w, out_f32=out_f32)
    assert y.dtype == (torch.float32 if out_f32 else torch.bfloat16) and y.shape == (T, N_)
    want = R.linear(x.cpu(), LinearWeight(q, fp8_scale=s))
    assert ((y.float().cpu() - want).abs().max() / want.abs().max()).item() < 1e-2


@pytest.mark.gpu
def test_fp8_kept_engine_gpu_matches_oracle():
    from slopllm_b200.models.dense import assemble_dense_weights
    cfg = DenseConfig.tiny()
    q8, plain = _fp8_checkpoint(cfg)
    w = assemble_dense_weights(cfg, q8, "cuda", torch.bfloat16, keep_fp8=True)
    assert w.layers[0].w_qkv.is_fp8
    prompt = torch.randint(2, cfg.vocab_size, (150,), generator=torch.Generator().manual_seed(7)).tolist()
    errs = teacher_forced_errors(cfg, w, plain, "cuda", prompt, 4, chunk=64)
    assert max(errs) < 6e-2, errs
