"""Kernel micro-benchmarks at the production shapes of one rank of a TP-8 GLM-5-class model.

    python -m slopllm_b200.cli.kernel_bench [--cases linear,mlp,moe,gemm,fp8] [--tokens 1,8,32,4096] [--iters 20]

For every (kernel, token count) it prints one JSON line with the device time (CUDA events, median of `--iters`
runs, three warm-up runs, a 256 MB write between runs so that no operand is served from L2), the algorithmic
bytes and FLOPs, and both as fractions of the measured roofline (`MEASURED_PEAKS.json` in the working
directory, or `--peaks <file>`; otherwise 6650 GB/s and 1590 TFLOP/s and the line says "fallback").

The reference's counterparts are `tests/python/bench_gemv.py`, `tests/python/bench_nvfp4_mul_mat_id.py`,
`tests/python/bench_indexer_decode.py` and `tests/python/bench_indexer_prefill.py` (the attention / indexer
kernels are covered by `slopllm_b200.cli.profile_step --op-times`, which times them inside a real step).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
from typing import Callable, Dict, List, Tuple

import torch

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def load_peaks(path: str | None = None) -> Dict[str, float]:
    """Roofline denominators: measured copy bandwidth (GB/s) and bf16 GEMM throughput (TFLOP/s)."""
    for p in ([path] if path else []) + ["MEASURED_PEAKS.json"]:
        if p and os.path.exists(p):
            with open(p) as f:
                d = json.load(f)
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
    return dict(FALLBACK_PEAKS)


def roofline_row(name: str, tokens: int, us: float, nbytes: float, flops: float, peaks: Dict[str, float]) -> Dict:
    """One result line: achieved bandwidth / throughput and the fraction of the slower-bound roofline."""
    t_mem = nbytes / (peaks["hbm_gbs"] * 1e9)
    t_mma = flops / (peaks["bf16_tflops"] * 1e12)
    bound = "memory" if t_mem >= t_mma else "tensor"
    floor_us = 1e6 * max(t_mem, t_mma)
    return {"kernel": name, "tokens": tokens, "us": round(us, 2), "gbytes_s": round(nbytes / us / 1e3, 1),
            "tflops": round(flops / us / 1e6, 2), "bound": bound, "roofline_us": round(floor_us, 2),
            "fraction_of_roofline": round(floor_us / us, 3), "peaks": peaks["source"]}


def linear_shapes(cfg, tp: int) -> List[Tuple[str, int, int, bool]]:
    """(name, out features, in features, nvfp4) of one rank's linears."""
    hl = cfg.num_attention_heads // tp
    qkv_rows = cfg.q_lora_rank + cfg.kv_lora_rank + cfg.qk_rope_head_dim + cfg.index_head_dim + cfg.index_n_heads
    qb_rows = hl * (cfg.qk_nope_head_dim + cfg.qk_rope_head_dim) + cfg.index_n_heads * cfg.index_head_dim
    return [
        ("qkv_a_bf16", qkv_rows, cfg.hidden_size, False),
        ("q_b_bf16", qb_rows, cfg.q_lora_rank, False),
        ("o_proj", cfg.hidden_size, hl * cfg.v_head_dim, bool(cfg.quant_o_proj)),
        ("dense_gate_up", 2 * cfg.intermediate_size // tp, cfg.hidden_size, bool(cfg.quant_dense_mlp)),
        ("dense_down", cfg.hidden_size, cfg.intermediate_size // tp, bool(cfg.quant_dense_mlp)),
        ("lm_head_bf16", cfg.vocab_size // tp, cfg.hidden_size, False),
    ]


def weight_bytes(n: int, k: int, nvfp4: bool) -> int:
    return n * k // 2 + n * k // 16 if nvfp4 else 2 * n * k


def time_op(fn: Callable[[], object], iters: int, flush: torch.Tensor) -> float:
    """Median device time in microseconds; `flush` (larger than L2) is rewritten before every timed run."""
    for _ in range(3):
        fn()
    times = []
    for _ in range(iters):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        times.append(1e3 * a.elapsed_time(b))
    return statistics.median(times)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="slopllm_b200.cli.kernel_bench")
    ap.add_argument("--cases", default="linear,mlp,moe")
    ap.add_argument("--tokens", default="1,8,32,4096")
    ap.add_argument("--tp-shape", type=int, default=8)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--peaks", default=None)
    args = ap.parse_args(argv)
    from ..config import GlmMoeDsaConfig
    from ..models.weights import _gen, _rand_linear, random_layer
    from ..ops.cuda_ops import CudaOps
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks = load_peaks(args.peaks)
    cfg = GlmMoeDsaConfig.glm5(num_layers=4)
    ops = CudaOps(cfg)
    tokens = [int(t) for t in args.tokens.split(",")]
    cases = set(args.cases.split(","))
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    g = _gen(1, dev)
    rows = []

    def emit(r):
        rows.append(r)
        print(json.dumps(r), flush=True)

    if "linear" in cases:
        for name, n, k, fp4 in linear_shapes(cfg, args.tp_shape):
            w = _rand_linear(n, k, g, dev, torch.bfloat16, fp4)
            for T in tokens:
                x = torch.randn(T, k, device=dev, generator=g).to(torch.bfloat16)
                us = time_op(lambda: ops.linear(x, w), args.iters, flush)
                emit(roofline_row(name + ("_nvfp4" if fp4 else ""), T, us, weight_bytes(n, k, fp4) + 2 * T * (n + k), 2.0 * T * n * k, peaks))
            del w
    if "gemm" in cases:
        # the tcgen05 GEMM itself (bf16 weights of every linear's shape) at both tile widths, and the two grouped expert
        # GEMMs of a prefill chunk (rows sorted by expert, 8 routes per token)
        from ..ops import tcgen05
        from ..ops.gemm import grouped_gemm
        for T in [t for t in tokens if t > 32]:
            for name, n, k, _ in linear_shapes(cfg, args.tp_shape):
                w = (torch.randn(n, k, device=dev, generator=g) * 0.02).to(torch.bfloat16)
                x = torch.randn(T, k, device=dev, generator=g).to(torch.bfloat16)
                for bn in (128, 256):
                    us = time_op(lambda: tcgen05.gemm_bf16(x, w, False, bn), args.iters, flush)
                    emit(roofline_row(f"gemm_bn{bn}_{name}", T, us, 2.0 * (n * k + T * (n + k)), 2.0 * T * n * k, peaks))
                del w, x
            E, I, Hh = cfg.n_routed_experts, cfg.moe_intermediate_size // args.tp_shape, cfg.hidden_size
            nrows = T * cfg.num_experts_per_tok
            cnt = torch.bincount(torch.randint(0, E, (nrows,), device=dev, generator=g), minlength=E)
            off = torch.zeros(E + 1, dtype=torch.int32, device=dev)
            off[1:] = torch.cumsum(cnt, 0).to(torch.int32)
            for name, n, k in (("grouped_gate_up", 2 * I, Hh), ("grouped_down", Hh, I)):
                w = (torch.randn(E, n, k, device=dev, generator=g) * 0.02).to(torch.bfloat16)
                a = torch.randn(nrows, k, device=dev, generator=g).to(torch.bfloat16)
                for bn in (128, 256):
                    us = time_op(lambda: grouped_gemm(a, w, off, False, bn), args.iters, flush)
                    emit(roofline_row(f"{name}_bn{bn}", T, us, 2.0 * (E * n * k + nrows * (n + k)), 2.0 * nrows * n * k, peaks))
                del w, a
    if "fp8" in cases:
        # FP8 block-scaled projections of a Qwen3-8B-class dense model kept in FP8 (one byte per weight streamed)
        from ..models.weights import LinearWeight
        from ..ops import dense as D
        for name, n, k in (("fp8_qkv", 6144, 4096), ("fp8_o_proj", 4096, 4096), ("fp8_gate_up", 24576, 4096), ("fp8_down", 4096, 12288)):
            q, sc = D.fp8_block_quantize(torch.randn(n, k, device=dev, generator=g) * 0.05)
            w = LinearWeight(q, fp8_scale=sc)
            for T in tokens:
                x = torch.randn(T, k, device=dev, generator=g).to(torch.bfloat16)
                us = time_op(lambda: ops.linear(x, w), args.iters, flush)
                emit(roofline_row(name, T, us, n * k + 4 * sc.numel() + 2 * T * (n + k), 2.0 * T * n * k, peaks))
            del w, q
    H = cfg.hidden_size
    if "mlp" in cases:
        lw = random_layer(cfg, 0, 0, dev, torch.bfloat16, 0, args.tp_shape, exact=False)
        nb = lw.mlp_w13.nbytes() + lw.mlp_w2.nbytes()
        nk = lw.mlp_w13.out_features * lw.mlp_w13.in_features + lw.mlp_w2.out_features * lw.mlp_w2.in_features
        for T in tokens:
            x = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
            us = time_op(lambda: ops.dense_mlp(x, lw), args.iters, flush)
            emit(roofline_row("dense_mlp_layer", T, us, nb + 4 * T * H, 2.0 * T * nk, peaks))
        del lw
    if "moe" in cases:
        lw = random_layer(cfg, 3, 0, dev, torch.bfloat16, 0, args.tp_shape, exact=False)
        ex = lw.experts
        E = ex.w13.shape[0]
        per_expert = (ex.w13.numel() + ex.w2.numel() + ex.s13.numel() + ex.s2.numel()) // E if ex.is_nvfp4 else 2 * (ex.w13.numel() + ex.w2.numel()) // E
        per_expert_mac = (ex.w13.shape[1] * H + H * ex.inter)
        shared = 0 if lw.shared is None else per_expert * lw.shared.inter // ex.inter
        for T in tokens:
            x = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
            ids, _ = ops.route(x, lw)
            uniq = int(torch.unique(ids).numel())
            us = time_op(lambda: ops.moe_tp(x, lw), args.iters, flush)
            nbytes = uniq * per_expert + shared + lw.router_w.numel() * 2 + 4 * T * H
            flops = 2.0 * T * (cfg.num_experts_per_tok + (1 if lw.shared is not None else 0)) * per_expert_mac + 2.0 * T * E * H
            r = roofline_row("moe_layer", T, us, nbytes, flops, peaks)
            r["experts_touched"] = uniq
            emit(r)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
