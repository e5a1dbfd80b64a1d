"""Entry points on the CPU reference ops with random tiny models: argument handling, registry
checks and the evaluation / benchmark tools end to end (reference: `src/model_cli.ts`,
`src/run_*.ts`, `src/mtp_stats.ts`, `src/model_registry.ts`, `src/model_path.ts`)."""
import io
import json
import os
from contextlib import redirect_stdout

import pytest

from slopllm_b200.cli import mtp_bench, nll, prefill_bench, sweep
from slopllm_b200.models import registry
from slopllm_b200.utils.model_path import ModelNotFoundError, list_safetensors_shards, resolve_model_path
from slopllm_b200.utils.mtp_stats import MtpStats


def run_tool(mod, argv):
    buf = io.StringIO()
    with redirect_stdout(buf):
        assert mod.main(argv) == 0
    return [json.loads(l) for l in buf.getvalue().splitlines() if l.startswith("{")]


BASE = ["--cpu", "--random-init", "tiny", "--no-cuda-graph", "--batch-size", "2", "--chunk-size", "64", "--max-pages", "32"]


def test_prefill_bench_and_sweep():
    out = run_tool(prefill_bench, BASE + ["--contexts", "100,200"])
    assert [o["context"] for o in out] == [100, 200] and all(o["prefill_tok_s"] > 0 for o in out)
    out = run_tool(sweep, BASE + ["--batches", "1,2", "--contexts", "70", "--steps", "3", "--warmup", "1"])
    assert [(o["batch"], o["context"]) for o in out] == [(1, 70), (2, 70)]


def test_nll_tool(tmp_path):
    ids = [(7 * i + 3) % 500 for i in range(150)]
    p = tmp_path / "ids.json"
    p.write_text(json.dumps(ids))
    out = run_tool(nll, BASE + ["--ids-file", str(p), "--window", "64"])[0]
    assert out["tokens"] == 149 and out["ppl"] > 1.0


def test_mtp_bench_and_stats():
    out = run_tool(mtp_bench, BASE + ["--mtp", "2", "--context", "80", "--steps", "4", "--warmup", "1"])[0]
    assert out["drafts"] == 2 and out["sequence_steps"] == 8 and 1.0 <= out["accept_length"] <= 3.0
    s = MtpStats(3)
    s.record([[1, 2, 3, 4], [5], [6, 7]])
    assert s.accept_length == pytest.approx(7 / 3) and s.per_position_rates() == [pytest.approx(2 / 3), 0.5, 1.0]
    assert s.summary()["histogram"] == {"1": 1, "2": 1, "4": 1}


def test_dense_family_through_cli():
    out = run_tool(prefill_bench, ["--cpu", "--random-init", "qwen35-tiny", "--no-cuda-graph", "--batch-size", "2", "--chunk-size", "64",
                                   "--max-pages", "32", "--contexts", "90"])
    assert out[0]["context"] == 90


def test_registry_checks(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps({"model_type": "qwen3"}))
    mt, reg, _ = registry.inspect_model(str(tmp_path))
    assert mt == "qwen3" and not reg.mtp
    with pytest.raises(ValueError, match="does not support --cp"):
        registry.inspect_model(str(tmp_path), cp=True)
    with pytest.raises(ValueError, match="does not support --mtp"):
        registry.inspect_model(str(tmp_path), mtp=3)
    (tmp_path / "config.json").write_text(json.dumps({"model_type": "llama"}))
    with pytest.raises(ValueError, match="unsupported model_type"):
        registry.inspect_model(str(tmp_path))


def test_model_path_resolution(tmp_path, monkeypatch):
    monkeypatch.setenv("HF_HOME", str(tmp_path))
    with pytest.raises(ModelNotFoundError):
        resolve_model_path("org/name")
    base = tmp_path / "hub" / "models--org--name"
    (base / "refs").mkdir(parents=True)
    (base / "refs" / "main").write_text("abc123\n")
    with pytest.raises(ModelNotFoundError, match="snapshot"):
        resolve_model_path("org/name")
    snap = base / "snapshots" / "abc123"
    snap.mkdir(parents=True)
    assert resolve_model_path("org/name") == str(snap)
    assert resolve_model_path(str(snap)) == str(snap)
    with pytest.raises(FileNotFoundError):
        list_safetensors_shards(str(snap))
    (snap / "b.safetensors").write_bytes(b"")
    (snap / "a.safetensors").write_bytes(b"")
    assert [os.path.basename(p) for p in list_safetensors_shards(str(snap))] == ["a.safetensors", "b.safetensors"]
    (snap / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"x": "b.safetensors", "y": "b.safetensors", "z": "a.safetensors"}}))
    assert [os.path.basename(p) for p in list_safetensors_shards(str(snap))] == ["b.safetensors", "a.safetensors"]


def test_serve_entry_point_end_to_end():
    """`python -m slopllm_b200 serve` on the CPU ops with a random tiny model: health, model list, one completion."""
    import subprocess
    import sys
    import time
    import urllib.request
    from mp_util import _free_port
    port = _free_port()
    proc = subprocess.Popen([sys.executable, "-m", "slopllm_b200", "serve", "--cpu", "--random-init", "tiny", "--no-cuda-graph",
                             "--batch-size", "2", "--chunk-size", "64", "--max-pages", "32", "--port", str(port), "--no-warmup",
                             "--temperature", "0"], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    try:
        ok = False
        for _ in range(120):
            try:
                with urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=2) as r:
                    ok = r.status == 200
                    break
            except Exception:  # noqa: BLE001
                if proc.poll() is not None:
                    break
                time.sleep(0.5)
        assert ok, proc.stdout.read() if proc.poll() is not None else "server did not come up"
        with urllib.request.urlopen(f"http://127.0.0.1:{port}/v1/models", timeout=10) as r:
            assert json.loads(r.read())["data"][0]["id"] == "tiny"
        body = json.dumps({"model": "tiny", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 4}).encode()
        req = urllib.request.Request(f"http://127.0.0.1:{port}/v1/chat/completions", data=body, headers={"Content-Type": "application/json"})
        with urllib.request.urlopen(req, timeout=120) as r:
            out = json.loads(r.read())
        assert out["usage"]["completion_tokens"] >= 1 and out["choices"][0]["finish_reason"] in ("length", "stop")
    finally:
        proc.terminate()
        try:
            proc.wait(timeout=20)
        except subprocess.TimeoutExpired:
            proc.kill()


def test_kernel_bench_roofline_rows(tmp_path):
    from slopllm_b200.cli import kernel_bench as kb
    from slopllm_b200.config import GlmMoeDsaConfig
    peaks = kb.load_peaks(str(tmp_path / "missing.json")) if not (tmp_path / "x").exists() else None
    (tmp_path / "p.json").write_text('{"hbm_gbs": 6000.0, "bf16_tflops": 1500.0}')
    peaks = kb.load_peaks(str(tmp_path / "p.json"))
    assert peaks == {"hbm_gbs": 6000.0, "bf16_tflops": 1500.0, "source": "measured"}
    # 6 MB in 2 us = 3000 GB/s = half of the memory roofline; the FLOPs are negligible
    r = kb.roofline_row("k", 1, 2.0, 6e6, 1e6, peaks)
    assert r["bound"] == "memory" and abs(r["fraction_of_roofline"] - 0.5) < 1e-3 and r["gbytes_s"] == 3000.0
    r = kb.roofline_row("k", 4096, 100.0, 1e6, 1.5e11, peaks)
    assert r["bound"] == "tensor" and abs(r["fraction_of_roofline"] - 1.0) < 1e-3
    shapes = dict((n, (o, i, q)) for n, o, i, q in kb.linear_shapes(GlmMoeDsaConfig.glm5(num_layers=4), 8))
    assert shapes["o_proj"][0] == 6144 and shapes["lm_head_bf16"][1] == 6144
    assert kb.weight_bytes(128, 256, True) == 128 * 256 // 2 + 128 * 256 // 16


def test_op_timers_wrap_and_restore():
    from slopllm_b200.utils.tracing import OpTimers

    class Ops:
        name = "x"

        def add(self, a, b):
            return a + self.twice(b)

        def twice(self, b):
            return 2 * b

    ops = Ops()
    t = OpTimers(ops)
    assert ops.add(1, 2) == 5
    assert t.summary() == [] or all(r["calls"] >= 1 for r in t.summary())     # no CUDA: nothing recorded
    t.restore()
    assert ops.add.__func__ is Ops.add


def test_weights_doc_groups_layers_and_experts(tmp_path):
    import json
    import torch
    from slopllm_b200.checkpoint.safetensors_io import save_file
    from slopllm_b200.cli import weights_doc
    t = {"model.embed_tokens.weight": torch.zeros(8, 4, dtype=torch.bfloat16)}
    for layer in range(3):
        t[f"model.layers.{layer}.input_layernorm.weight"] = torch.zeros(4, dtype=torch.bfloat16)
        for e in range(2):
            t[f"model.layers.{layer}.mlp.experts.{e}.down_proj.weight"] = torch.zeros(4, 2, dtype=torch.uint8)
    save_file(t, str(tmp_path / "model-00001-of-00001.safetensors"))
    (tmp_path / "config.json").write_text(json.dumps({"model_type": "glm_moe_dsa", "num_hidden_layers": 2}))
    out = tmp_path / "w.md"
    assert weights_doc.main(["--model", str(tmp_path), "--output", str(out)]) == 0
    text = out.read_text()
    assert "| `model.layers.N.mlp.experts.E.down_proj.weight` | [4, 2] | U8 | 4 | 32 B |" in text
    assert "| `model.layers.MTP.mlp.experts.E.down_proj.weight` **MTP** | [4, 2] | U8 | 2 | 16 B |" in text
    assert "**Total tensors**: 10" in text


def test_arena_flag_is_a_per_process_allocation_cap():
    import torch
    from slopllm_b200.cli.model_cli import apply_arena_cap, arena_fraction
    total = 180 << 30
    assert arena_fraction(0.0, total) == 1.0 and arena_fraction(360.0, total) == 1.0
    assert abs(arena_fraction(90.0, total) - 0.5) < 1e-9
    assert apply_arena_cap(torch.device("cpu"), 90.0) == 1.0          # nothing to cap on the CPU


def test_fused_switch_selects_library_collectives(monkeypatch):
    """`make_comm` gives the plain communicator on CPU, for one rank, with fused=False and with SLOPLLM_B200_FUSED=0."""
    import torch
    from slopllm_b200.parallel import fused as F
    from slopllm_b200.parallel.dist import Comm, ParallelContext
    assert type(F.make_comm(ParallelContext())) is Comm
    made = []

    class FakeNvlink(Comm):
        def __init__(self, ctx, cfg):
            super().__init__(ctx)
            made.append(ctx)
    import slopllm_b200.parallel.nvlink as NV
    monkeypatch.setattr(NV, "NvlinkComm", FakeNvlink)
    ctx = ParallelContext(0, 2, torch.device("cuda", 0))
    assert type(F.make_comm(ctx)) is FakeNvlink and len(made) == 1
    assert type(F.make_comm(ctx, fused=False)) is Comm
    monkeypatch.setenv("SLOPLLM_B200_FUSED", "0")
    assert type(F.make_comm(ctx)) is Comm and len(made) == 1


def test_generation_defaults_from_the_checkpoint(tmp_path):
    """Flags win, then generation_config.json, then config.json, then the built-in values."""
    import json
    from types import SimpleNamespace
    from slopllm_b200.cli.serve import BUILTIN_SAMPLING, parse_args
    from slopllm_b200.utils.generation_config import (apply_generation_defaults, load_generation_defaults,
                                                      max_position_embeddings)
    (tmp_path / "config.json").write_text(json.dumps({"temperature": 0.9, "top_k": 50, "max_position_embeddings": 202752,
                                                      "repetition_penalty": None}))
    (tmp_path / "generation_config.json").write_text(json.dumps({"temperature": 1.0, "top_p": 0.8, "do_sample": True}))
    d = load_generation_defaults(str(tmp_path))
    assert d == {"temperature": 1.0, "top_p": 0.8, "top_k": 50}
    assert max_position_embeddings(str(tmp_path)) == 202752 and max_position_embeddings(None) is None
    (tmp_path / "mm").mkdir()
    (tmp_path / "mm" / "config.json").write_text(json.dumps({"text_config": {"max_position_embeddings": 4096}}))
    assert max_position_embeddings(str(tmp_path / "mm")) == 4096
    args = parse_args(["--random-init", "tiny", "--top-p", "0.5"])
    assert args.temperature is None and args.top_p == 0.5
    origin = apply_generation_defaults(args, str(tmp_path), BUILTIN_SAMPLING)
    assert (args.temperature, args.top_p, args.top_k, args.repetition_penalty, args.max_tokens) == (1.0, 0.5, 50, 1.0, 65536)
    assert origin == {"temperature": "checkpoint", "top_p": "flag", "top_k": "checkpoint", "repetition_penalty": "default",
                      "max_tokens": "default"}
    bare = SimpleNamespace(temperature=None, top_p=None, top_k=None, repetition_penalty=None, max_tokens=None)
    apply_generation_defaults(bare, None, BUILTIN_SAMPLING)
    assert (bare.temperature, bare.top_p, bare.top_k) == (0.6, 0.95, 20)


def test_memory_plan_matches_real_weights_and_caches():
    """The analytic sizing against weights and caches that were really built (tiny and a mid-size shape, TP 1 / 2, experts
    split by column or by expert), then the plan arithmetic and the `plan` command."""
    import json
    import torch
    from slopllm_b200.cli import plan as plan_cli
    from slopllm_b200.config import GlmMoeDsaConfig
    from slopllm_b200.models.glm_moe_dsa import KVCacheTensors
    from slopllm_b200.models.weights import random_model
    from slopllm_b200.utils.sizing import GIB, kv_page_bytes, model_weight_bytes, plan_memory
    mid = GlmMoeDsaConfig(hidden_size=512, intermediate_size=1024, moe_intermediate_size=256, num_hidden_layers=3,
                          num_nextn_predict_layers=1, vocab_size=2048, num_attention_heads=8, q_lora_rank=256,
                          n_routed_experts=16, num_experts_per_tok=4, n_group=4, topk_group=2, index_topk=64,
                          first_k_dense_replace=1, quant_o_proj=True, quant_dense_mlp=True)
    for cfg in (GlmMoeDsaConfig.tiny(), mid):
        for tp, ep in ((1, False), (2, False), (2, True)):
            w = random_model(cfg, 0, "cpu", torch.bfloat16, 0, tp, ep=ep, with_mtp=True)
            est = model_weight_bytes(cfg, tp, ep, True)
            assert abs(est - w.nbytes()) <= 0.002 * w.nbytes(), (tp, ep, est, w.nbytes())
        assert KVCacheTensors.allocate(cfg, 4, "cpu").nbytes() == 4 * kv_page_bytes(cfg, True)
    glm5 = GlmMoeDsaConfig.glm5(78)
    p8 = plan_memory(glm5, world=8, cp=True, mtp=3, max_pages=8192)
    assert 50 * GIB < p8.weights_bytes < 60 * GIB and p8.tokens_per_page == 512 and p8.requested_fits
    assert p8.max_pages == (p8.budget_bytes - p8.weights_bytes - p8.workspace_bytes) // p8.page_bytes
    p1 = plan_memory(glm5, world=1)
    assert p1.weights_bytes > 180 * GIB and p1.max_pages == 0 and not p1.requested_fits      # the model needs several GPUs
    small = plan_memory(glm5, world=8, arena_gb=70.0, max_pages=8192)
    assert small.max_pages < 8192 and not small.requested_fits
    assert plan_cli.main(["--random-init", "glm5", "--world", "8", "--cp", "--mtp", "--max-pages", "8192"]) == 0
    assert plan_cli.main(["--random-init", "glm5", "--world", "1"]) == 1
    assert json.dumps(p8.to_dict())


def test_memory_plan_for_dense_families():
    import torch
    from slopllm_b200.cli import plan as plan_cli
    from slopllm_b200.models.dense import DenseCache, DenseConfig, random_dense_model
    from slopllm_b200.runtime.workspace import walk_tensors
    from slopllm_b200.utils.sizing import dense_kv_page_bytes, dense_weight_bytes, plan_dense
    for hybrid in (False, True):
        cfg = DenseConfig.tiny(hybrid=hybrid)
        for tp in (1, 2):
            w, _ = random_dense_model(cfg, 0, "cpu", torch.bfloat16, 0, tp)
            seen, total = set(), [0]

            def add(t):
                if t.data_ptr() not in seen:
                    seen.add(t.data_ptr())
                    total[0] += t.numel() * t.element_size()
            walk_tensors(w, add)
            assert dense_weight_bytes(cfg, tp) == total[0], (hybrid, tp)
            c = DenseCache(cfg, 4, "cpu", tp=tp)
            kv = sum(x.numel() * x.element_size() for x in list(c.k.values()) + list(c.v.values()))
            assert kv == 4 * dense_kv_page_bytes(cfg, tp)
    p = plan_dense(DenseConfig.tiny(), world=1, max_pages=64)
    assert p.requested_fits and p.tokens_per_page == 64 and p.max_pages > 64
    assert dense_weight_bytes(DenseConfig.tiny(), 1, fp8=True) < dense_weight_bytes(DenseConfig.tiny(), 1)
    assert plan_cli.main(["--random-init", "qwen3", "--max-pages", "64"]) == 0
