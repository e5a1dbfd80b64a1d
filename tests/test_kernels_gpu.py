"""Each sm_100a kernel against the plain PyTorch fp32 reference of the same op.

Tolerances follow the reference's kernel tests (ATOL = RTOL = 1e-2 on bf16 data,
`tests/python/helpers.py`), relative to the magnitude of the expected output.
"""
import math

import pytest
import torch

from slopllm_b200.config import GlmMoeDsaConfig
from slopllm_b200.models.glm_moe_dsa import KVCacheTensors, StepState
from slopllm_b200.models.weights import LinearWeight, random_layer
from slopllm_b200.ops import RefOps, quant, reference as R

pytestmark = pytest.mark.gpu
DEV = "cuda"


def close(a, b, tol=1e-2, what=""):
    a, b = a.to(torch.float32), b.to(torch.float32)
    assert a.shape == b.shape, (what, a.shape, b.shape)
    scale = b.abs().max().clamp(min=1e-6)
    err = ((a - b).abs().max() / scale).item()
    assert err <= tol, f"{what}: max rel-to-peak error {err:.4g} > {tol}"


def cuda_ops(cfg):
    from slopllm_b200.ops.cuda_ops import CudaOps
    return CudaOps(cfg)


def mini_cfg(**kw):
    """GLM-5 head geometry with a small hidden size and few experts."""
    base = dict(hidden_size=1024, intermediate_size=1024, moe_intermediate_size=256, num_hidden_layers=2,
                num_nextn_predict_layers=1, vocab_size=4096, num_attention_heads=8, q_lora_rank=512, kv_lora_rank=512,
                qk_nope_head_dim=192, qk_rope_head_dim=64, v_head_dim=256, n_routed_experts=16, n_shared_experts=1,
                num_experts_per_tok=4, n_group=4, topk_group=2, index_topk=256, index_head_dim=128, index_n_heads=32,
                first_k_dense_replace=1, quant_o_proj=True, quant_dense_mlp=True)
    base.update(kw)
    return GlmMoeDsaConfig(**base)


@pytest.mark.parametrize("T", [1, 2, 3, 5, 8, 19, 32])
@pytest.mark.parametrize("N,K", [(256, 512), (2784, 6144), (1000, 2048), (256, 6144)])
def test_gemv_bf16(T, N, K):
    g = torch.Generator(device=DEV).manual_seed(T * 7 + N)
    x = torch.randn(T, K, device=DEV, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV, generator=g) * 0.05).to(torch.bfloat16)
    ops = cuda_ops(GlmMoeDsaConfig.tiny())
    for f32 in (False, True):
        y = ops.linear(x, LinearWeight(w), out_f32=f32)
        close(y, x.float() @ w.float().t(), what=f"gemv_bf16 T={T} f32={f32}")


@pytest.mark.parametrize("T", [1, 2, 4, 7, 16, 23, 32])
@pytest.mark.parametrize("N,K", [(512, 256), (6144, 2048), (4096, 6144), (1000, 128)])
def test_gemv_nvfp4(T, N, K):
    g = torch.Generator(device=DEV).manual_seed(T + K)
    x = torch.randn(T, K, device=DEV, generator=g).to(torch.bfloat16)
    w = LinearWeight(*quant.random_nvfp4((N, K), g, DEV))
    w.scale2.fill_(0.37)
    ops = cuda_ops(GlmMoeDsaConfig.tiny())
    y = ops.linear(x, w, out_f32=True)
    close(y, R.linear(x, w), what=f"gemv_nvfp4 T={T}")
    close(ops.linear(x, w), R.linear(x, w), what=f"gemv_nvfp4 bf16 out T={T}")
    from slopllm_b200.ops import tcgen05
    torch.cuda.synchronize()
    tcgen05.check_errors(DEV)


def test_nvfp4_roundtrip_quantize():
    g = torch.Generator(device=DEV).manual_seed(3)
    w = torch.randn(64, 256, device=DEV, generator=g)
    p, s, gs = quant.nvfp4_quantize(w)
    wd = quant.nvfp4_dequantize(p, s, gs)
    assert ((wd - w).abs().mean() / w.abs().mean()).item() < 0.12


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 384, 512), (300, 200, 1024), (1000, 2784, 6144), (4096, 6144, 2048)])
@pytest.mark.parametrize("bn", [64, 128, 256])
def test_gemm_tcgen05(M, N, K, bn):
    from slopllm_b200.ops import tcgen05
    g = torch.Generator(device=DEV).manual_seed(M + N)
    a = torch.randn(M, K, device=DEV, generator=g).to(torch.bfloat16)
    b = (torch.randn(N, K, device=DEV, generator=g) * 0.05).to(torch.bfloat16)
    for f32 in (True, False):
        y = tcgen05.gemm_bf16(a, b, f32, bn=bn)
        torch.cuda.synchronize()
        tcgen05.check_errors(DEV)
        close(y, a.float() @ b.float().t(), tol=1e-2, what=f"tcgen05 gemm {M}x{N}x{K} bn={bn} f32={f32}")


def test_add_rmsnorm_and_embed():
    cfg = GlmMoeDsaConfig.tiny()
    ops, ref = cuda_ops(cfg), RefOps(cfg)
    g = torch.Generator(device=DEV).manual_seed(0)
    H = 6144
    table = torch.randn(100, H, device=DEV, generator=g).to(torch.bfloat16)
    ids = torch.tensor([3, 99, 0, 7], device=DEV)
    assert torch.equal(ops.embed(ids, table), table[ids])
    x = torch.randn(5, H, device=DEV, generator=g)
    res = torch.randn(5, H, device=DEV, generator=g)
    w = torch.rand(H, device=DEV, generator=g).to(torch.bfloat16)
    for xin in (x, x.to(torch.bfloat16)):
        o, r = ops.add_rmsnorm(xin, res, w)
        eo, er = ref.add_rmsnorm(xin, res, w)
        close(o, eo, what="add_rmsnorm out")
        close(r, er, tol=1e-5, what="residual")
    o, r = ops.add_rmsnorm(x, None, w)
    close(o, ref.add_rmsnorm(x, None, w)[0], what="rmsnorm first")


def _state(cfg, positions, batch_idx, n_pages_per_seq, B, cp_world=1, cp_rank=0):
    pt = torch.arange(B * n_pages_per_seq, dtype=torch.int32, device=DEV).reshape(B, n_pages_per_seq)
    # shuffle physical pages so that logical != physical
    perm = torch.randperm(B * n_pages_per_seq, device=DEV, generator=torch.Generator(device=DEV).manual_seed(5))
    pt = perm[pt.to(torch.int64)].to(torch.int32)
    pos = torch.tensor(positions, dtype=torch.int32, device=DEV)
    return StepState(input_ids=torch.zeros(len(positions), dtype=torch.int64, device=DEV), positions=pos,
                     batch_idx=torch.tensor(batch_idx, dtype=torch.int32, device=DEV), page_table=pt,
                     cp_world=cp_world, cp_rank=cp_rank, max_kv_len=max(positions) + 1)


@pytest.mark.parametrize("which", ["tiny", "mini"])
@pytest.mark.parametrize("cp", [(1, 0), (2, 1)])
def test_attn_pre_and_q_post(which, cp):
    cfg = GlmMoeDsaConfig.tiny() if which == "tiny" else mini_cfg()
    ops, ref = cuda_ops(cfg), RefOps(cfg)
    lw = random_layer(cfg, 1 if which == "tiny" else 0, 0, DEV, torch.bfloat16)
    T = 6
    st = _state(cfg, [0, 1, 130, 131, 5, 64], [0, 0, 0, 0, 1, 1], 4, 2, *cp)
    g = torch.Generator(device=DEV).manual_seed(1)
    x = torch.randn(T, cfg.hidden_size, device=DEV, generator=g).to(torch.bfloat16)
    qkv = ref.linear(x, lw.w_qkv_a).to(torch.bfloat16)
    c1 = KVCacheTensors.allocate(cfg, 8, DEV, 1).layers[0]
    c2 = KVCacheTensors.allocate(cfg, 8, DEV, 1).layers[0]
    if c1.idx is None:
        c1.idx = torch.zeros(8 * 64, cfg.index_row_bytes, dtype=torch.uint8, device=DEV)
        c2.idx = torch.zeros_like(c1.idx)
    cq, iw = ops.attn_pre(qkv, lw, st, c1)
    ecq, eiw = ref.attn_pre(qkv, lw, st, c2)
    close(cq, ecq, what="c_q")
    close(iw, eiw, what="idx_w")
    a, b = quant.unpack_kv_rows(c1.kv, cfg.kv_lora_rank, cfg.qk_rope_head_dim, cfg.kv_quant_group)
    ea, eb = quant.unpack_kv_rows(c2.kv, cfg.kv_lora_rank, cfg.qk_rope_head_dim, cfg.kv_quant_group)
    close(a, ea, tol=7e-2, what="ckv rows")      # one e4m3 step at most
    close(b, eb, what="kpe rows")
    close(quant.unpack_index_rows(c1.idx, cfg.index_head_dim), quant.unpack_index_rows(c2.idx, cfg.index_head_dim),
          tol=7e-2, what="index rows")
    qb = ref.linear(ecq, lw.w_q_b).to(torch.bfloat16)
    qa, qp, q8, we = ops.q_post(qb, lw, st, iw)
    eqa, eqp, eq8, ewe = ref.q_post(qb, lw, st, eiw)
    close(qa, eqa, what="q_abs")
    close(qp, eqp, what="q_pe")
    got = q8.view(torch.float8_e4m3fn).float() * (we / (iw * cfg.index_head_dim ** -0.5)).unsqueeze(-1)
    exp = eq8 * (ewe / (eiw * cfg.index_head_dim ** -0.5)).unsqueeze(-1)
    close(got, exp, tol=7e-2, what="indexer q")


@pytest.mark.parametrize("E,k,ng,tg", [(256, 8, 8, 4), (256, 8, 1, 1), (8, 2, 1, 1), (16, 4, 4, 2)])
def test_route_topk(E, k, ng, tg):
    cfg = mini_cfg(n_routed_experts=E, num_experts_per_tok=k, n_group=ng, topk_group=tg, hidden_size=512)
    ops, ref = cuda_ops(cfg), RefOps(cfg)
    g = torch.Generator(device=DEV).manual_seed(E)
    lw = type("L", (), {})()
    lw.router_w = torch.randn(E, 512, device=DEV, generator=g).to(torch.bfloat16)
    lw.router_bias = torch.randn(E, device=DEV, generator=g) * 0.1
    x = torch.randn(9, 512, device=DEV, generator=g).to(torch.bfloat16)
    logits = ops._router_logits(x, lw)
    ids, w = ops.route(x, lw)
    eids, ew = R.moe_route(logits, lw.router_bias, k, ng, tg, True, cfg.routed_scaling_factor)
    assert torch.equal(ids.sort(1).values, eids.sort(1).values)
    close(w.gather(1, ids.argsort(1)), ew.gather(1, eids.argsort(1)), tol=1e-4, what="route weights")


def test_topk_to_slots():
    cfg = mini_cfg()
    ops, ref = cuda_ops(cfg), RefOps(cfg)
    st = _state(cfg, [300, 301, 17], [0, 0, 1], 8, 2, 2, 1)
    pos = torch.full((3, 256), -1, dtype=torch.int32, device=DEV)
    pos[0, :200] = torch.arange(0, 200, dtype=torch.int32, device=DEV) + 50
    pos[1, :256] = torch.arange(0, 256, dtype=torch.int32, device=DEV) + 40
    pos[2, :18] = torch.arange(18, dtype=torch.int32, device=DEV)
    for local_only in (False, True):
        s, l = ops.topk_to_slots(pos, st, local_only)
        es, el = ref.topk_to_slots(pos, st, local_only)
        assert torch.equal(l, el)
        assert torch.equal(s, es)


@pytest.mark.parametrize("which,ctx", [("tiny", 300), ("mini", 700), ("mini", 3000)])
@pytest.mark.parametrize("cp", [(1, 0), (4, 3)])
def test_indexer_topk(which, ctx, cp):
    cfg = GlmMoeDsaConfig.tiny() if which == "tiny" else mini_cfg()
    ops, ref = cuda_ops(cfg), RefOps(cfg)
    W, r = cp
    n_pages = -(-ctx // (64 * W)) + 1
    positions = [ctx - 1, ctx - 2, cfg.index_topk - 1, 10]
    st = _state(cfg, positions, [0, 0, 1, 1], n_pages, 2, W, r)
    g = torch.Generator(device=DEV).manual_seed(ctx)
    Di, Hi = cfg.index_head_dim, cfg.index_n_heads
    cache = type("C", (), {})()
    keys = torch.randn(2 * n_pages * 64, Di, device=DEV, generator=g)
    cache.idx = quant.pack_index_rows(keys)
    q = torch.randn(4, Hi, Di, device=DEV, generator=g)
    hw = torch.rand(4, Hi, device=DEV, generator=g)
    q8f, weff = R.indexer_quantize_q(q, hw, Di ** -0.5)
    q8 = q8f.to(torch.float8_e4m3fn).view(torch.uint8)
    pos, sc = ops.indexer_topk(q8, weff, cache, st)
    epos, esc = ref.indexer_topk(q8f, weff, cache, st)
    for t in range(4):
        a, b = set(pos[t][pos[t] >= 0].tolist()), set(epos[t][epos[t] >= 0].tolist())
        assert len(a) == len(b), (t, len(a), len(b))
        assert len(a ^ b) <= max(2, len(b) // 100), (t, len(a ^ b))      # ties at the threshold only
        valid = pos[t][pos[t] >= 0]
        assert torch.all(valid[1:] > valid[:-1])


@pytest.mark.parametrize("cp", [(1, 0), (2, 1)])
def test_indexer_prefill_tiles_match_per_token_kernel(cp):
    """More than 32 query rows take the prefill scorer (8 tokens per CTA share key pages in shared memory; a group that mixes
    sequences loads per warp): same selection as the fp32 reference, same positions and scores as the per-token kernel."""
    from slopllm_b200.ops import native as N
    cfg = mini_cfg()
    ops, ref = cuda_ops(cfg), RefOps(cfg)
    W, r = cp
    ctx = 1500
    n_pages = -(-ctx // (64 * W)) + 1
    positions = list(range(ctx - 36, ctx)) + [ctx - 1, 900, cfg.index_topk - 1, 10]        # 36 rows of sequence 0, 4 of sequence 1
    st = _state(cfg, positions, [0] * 36 + [1] * 4, n_pages, 2, W, r)
    g = torch.Generator(device=DEV).manual_seed(77)
    Di, Hi, T = cfg.index_head_dim, cfg.index_n_heads, len(positions)
    cache = type("C", (), {})()
    cache.idx = quant.pack_index_rows(torch.randn(2 * n_pages * 64, Di, device=DEV, generator=g))
    q = torch.randn(T, Hi, Di, device=DEV, generator=g)
    hw = torch.rand(T, Hi, device=DEV, generator=g)
    q8f, weff = R.indexer_quantize_q(q, hw, Di ** -0.5)
    q8 = q8f.to(torch.float8_e4m3fn).view(torch.uint8)
    pos, sc = ops.indexer_topk(q8, weff, cache, st)
    N.kernels().sl_indexer_set_tiled(0)
    try:
        st.extra.clear()
        pos2, sc2 = ops.indexer_topk(q8, weff, cache, st)
    finally:
        N.kernels().sl_indexer_set_tiled(1)
    assert torch.equal(pos, pos2) and torch.equal(sc, sc2)
    epos, _ = ref.indexer_topk(q8f, weff, cache, st)
    for t in range(T):
        a, b = set(pos[t][pos[t] >= 0].tolist()), set(epos[t][epos[t] >= 0].tolist())
        assert len(a) == len(b) and len(a ^ b) <= max(2, len(b) // 100), (t, len(a), len(b), len(a ^ b))


@pytest.mark.parametrize("cp,ctx,T", [((1, 0), 3000, 100), ((1, 0), 9000, 257), ((2, 1), 5000, 64), ((1, 0), 2049, 40)])
def test_indexer_prefill_scorer_on_tcgen05(cp, ctx, T):
    """A prefill chunk of one sequence takes the tensor-core scorer (keys on the 128 MMA rows, 8 tokens x 32 heads on the
    columns, relu / head weights / key scale folded per TMEM lane): same scores as the mma.sync kernels up to the order
    of the fp32 sums, same selection as the fp32 reference.  Ragged last token block and key tile, rows below the
    top-k threshold, logical != physical pages, a context-parallel rank."""
    from slopllm_b200.ops import native as N, tcgen05
    cfg = mini_cfg()
    ops, ref = cuda_ops(cfg), RefOps(cfg)
    W, r = cp
    n_pages = -(-ctx // (64 * W)) + 1
    positions = list(range(ctx - T, ctx))
    st = _state(cfg, positions, [0] * T, n_pages, 1, W, r)
    st.extra["one_sequence"] = True
    g = torch.Generator(device=DEV).manual_seed(ctx + T)
    Di, Hi = cfg.index_head_dim, cfg.index_n_heads
    assert (Di, Hi) == (128, 32)
    cache = type("C", (), {})()
    cache.idx = quant.pack_index_rows(torch.randn(n_pages * 64, Di, device=DEV, generator=g))
    q = torch.randn(T, Hi, Di, device=DEV, generator=g)
    hw = torch.rand(T, Hi, device=DEV, generator=g) - 0.3                  # some negative head weights
    q8f, weff = R.indexer_quantize_q(q, hw, Di ** -0.5)
    q8 = q8f.to(torch.float8_e4m3fn).view(torch.uint8)
    pos, sc = ops.indexer_topk(q8, weff, cache, st)
    scores_tc = st.extra["idx_scores"].clone()
    tcgen05.check_errors(DEV)
    N.kernels().sl_indexer_set_tcgen05(0)
    try:
        st.extra.pop("idx_scores")
        pos2, sc2 = ops.indexer_topk(q8, weff, cache, st)
        scores_mma = st.extra["idx_scores"]
    finally:
        N.kernels().sl_indexer_set_tcgen05(1)
    for t in range(T):
        p = positions[t]
        n_vis = ((p - r) // W + 1 if p >= r else 0) if p + 1 > cfg.index_topk else 0
        a, b = scores_tc[t, :n_vis], scores_mma[t, :n_vis]
        assert torch.allclose(a, b, rtol=1e-4, atol=1e-4 * float(b.abs().max() if n_vis else 1.0)), (t, n_vis)
    epos, _ = ref.indexer_topk(q8f, weff, cache, st)
    for t in range(T):
        a, b = set(pos[t][pos[t] >= 0].tolist()), set(epos[t][epos[t] >= 0].tolist())
        assert len(a) == len(b) and len(a ^ b) <= max(2, len(b) // 100), (t, len(a), len(b), len(a ^ b))


@pytest.mark.parametrize("T,h", [(100, 8), (257, 4), (4096, 8)])
def test_head_batched_products_on_tcgen05(T, h):
    """Prefill absorb (q_nope x W_kn per head, K = 192 taken from the 256-wide head slice of the projection) and value
    expansion (o x W_v per head) on the persistent tcgen05 GEMM with a per-head operand origin, against torch in fp32."""
    from slopllm_b200.ops import tcgen05
    cfg = mini_cfg(num_attention_heads=h)
    ops = cuda_ops(cfg)
    g = torch.Generator(device=DEV).manual_seed(T + h)
    Dn, Dr, Rr, Dv = cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.kv_lora_rank, cfg.v_head_dim
    qb = torch.randn(T, h * (Dn + Dr) + 64, device=DEV, generator=g).to(torch.bfloat16)      # wider than the heads (indexer columns)
    owner = type("L", (), {})()
    owner.w_kn = (torch.randn(h, Dn, Rr, device=DEV, generator=g) * 0.05).to(torch.bfloat16)
    q_abs = ops._head_batched_gemm(qb, Dn + Dr, Dn, owner, "w_kn")
    assert q_abs is not None and owner._w_kn_t.shape == (h * Rr, Dn)
    q_nope = qb[:, :h * (Dn + Dr)].view(T, h, Dn + Dr)[..., :Dn].float()
    want = torch.einsum("thd,hdr->thr", q_nope, owner.w_kn.float()).reshape(T, h * Rr)
    close(q_abs, want, tol=2e-2, what="absorb")
    o = (torch.randn(T, h, Rr, device=DEV, generator=g) * 0.3).to(torch.bfloat16)
    w_v = (torch.randn(h, Rr, Dv, device=DEV, generator=g) * 0.05).to(torch.bfloat16)
    out = ops.v_expand(o, w_v)
    assert getattr(w_v, "_sl_out_major", None) is not None
    close(out, torch.einsum("thr,hrv->thv", o.float(), w_v.float()).reshape(T, h * Dv), tol=2e-2, what="v_expand")
    close(ops.v_expand(o, w_v), out, tol=1e-6, what="second call (kept copy)")
    tcgen05.check_errors(DEV)


@pytest.mark.parametrize("which", ["tiny", "mini"])
def test_sparse_mla_and_v_expand(which):
    cfg = GlmMoeDsaConfig.tiny() if which == "tiny" else mini_cfg()
    ops, ref = cuda_ops(cfg), RefOps(cfg)
    g = torch.Generator(device=DEV).manual_seed(11)
    Rr, Dr, h, k = cfg.kv_lora_rank, cfg.qk_rope_head_dim, cfg.num_attention_heads, cfg.index_topk
    nslots = 1024
    cache = type("C", (), {})()
    cache.kv = quant.pack_kv_rows(torch.randn(nslots, Rr, device=DEV, generator=g),
                                  torch.randn(nslots, Dr, device=DEV, generator=g), cfg.kv_quant_group)
    T = 3
    q_abs = (torch.randn(T, h, Rr, device=DEV, generator=g) * 0.3).to(torch.bfloat16)
    q_pe = (torch.randn(T, h, Dr, device=DEV, generator=g) * 0.3).to(torch.bfloat16)
    slots = torch.full((T, k), -1, dtype=torch.int32, device=DEV)
    lengths = torch.tensor([k, 37, 0], dtype=torch.int32, device=DEV)
    for t in range(T):
        n = int(lengths[t])
        slots[t, :n] = torch.randperm(nslots, device=DEV, generator=g)[:n].to(torch.int32)
    o, lse = ops.sparse_mla(q_abs, q_pe, cache, slots, lengths)
    eo, elo = ref.sparse_mla(q_abs, q_pe, cache, slots, lengths)
    close(o, eo, what="sparse mla o")
    close(lse[:2], elo[:2], tol=1e-3, what="lse")
    assert torch.isinf(lse[2]).all()
    w_v = (torch.randn(h, Rr, cfg.v_head_dim, device=DEV, generator=g) * 0.05).to(torch.bfloat16)
    close(ops.v_expand(o, w_v), ref.v_expand(o, w_v), what="v_expand")


@pytest.mark.parametrize("h,T,q_scale", [(8, 3, 0.3), (8, 40, 4.0), (16, 3, 4.0), (12, 5, 0.3), (8, 320, 1.0), (40, 2, 1.0)])
def test_sparse_mla_keys_on_m(h, T, q_scale):
    """The keys-on-M sparse MLA kernel (kv_lora_rank a multiple of 128) at the production top-k: full, ragged and
    empty key lists, one or several key splits, 8 / 12 / 16 heads per CTA; `q_scale` 4 makes later chunks exceed the
    softmax reference of earlier ones (the rescale path); 320 rows need no key split, so the kernel writes the final
    output itself.  Also against the heads-on-M kernel through the switch."""
    from slopllm_b200.ops import native as N
    cfg = mini_cfg(num_attention_heads=h, index_topk=2048)
    ops, ref = cuda_ops(cfg), RefOps(cfg)
    g = torch.Generator(device=DEV).manual_seed(100 + h + T)
    Rr, Dr, k = cfg.kv_lora_rank, cfg.qk_rope_head_dim, cfg.index_topk
    nslots = 4096
    cache = type("C", (), {})()
    cache.kv = quant.pack_kv_rows(torch.randn(nslots, Rr, device=DEV, generator=g) * 2.0,
                                  torch.randn(nslots, Dr, device=DEV, generator=g), cfg.kv_quant_group)
    q_abs = (torch.randn(T, h, Rr, device=DEV, generator=g) * q_scale).to(torch.bfloat16)
    q_pe = (torch.randn(T, h, Dr, device=DEV, generator=g) * q_scale).to(torch.bfloat16)
    slots = torch.full((T, k), -1, dtype=torch.int32, device=DEV)
    lens = [k, 1000, 0, 65, 64, 1] + [k] * T
    lengths = torch.tensor(lens[:T], dtype=torch.int32, device=DEV)
    for t in range(T):
        n = int(lengths[t])
        slots[t, :n] = torch.randperm(nslots, device=DEV, generator=g)[:n].to(torch.int32)
    o, lse = ops.sparse_mla(q_abs, q_pe, cache, slots, lengths)
    eo, elo = ref.sparse_mla(q_abs, q_pe, cache, slots, lengths)
    live = lengths > 0
    close(o, eo, what="sparse mla o (keys on M)")
    close(lse[live], elo[live], tol=1e-3, what="lse (keys on M)")
    assert torch.isinf(lse[~live]).all() and (o[~live] == 0).all()
    N.kernels().sl_sparse_mla_set_transposed(0)
    try:
        o2, lse2 = ops.sparse_mla(q_abs, q_pe, cache, slots, lengths)
    finally:
        N.kernels().sl_sparse_mla_set_transposed(1)
    close(o, o2, tol=2e-2, what="keys-on-M vs heads-on-M")        # two approximations, each within 1e-2 of the fp32 definition
    close(lse[live], lse2[live], tol=1e-3, what="lse, keys-on-M vs heads-on-M")


@pytest.mark.parametrize("h,T,q_scale,kv_scale", [(8, 160, 1.0, 2.0), (8, 300, 4.0, 2.0), (16, 150, 1.0, 0.05), (4, 310, 0.3, 30.0),
                                                  (8, 200, 2.0, 1.0), (32, 80, 1.0, 1.0)])
def test_sparse_mla_prefill_on_tcgen05(h, T, q_scale, kv_scale):
    """Prefill-sized sparse MLA (no key split) runs on tcgen05 straight from the e4m3 cache rows: query and
    probabilities as two e4m3 terms, code tiles read K-major for the scores and MN-major for the values.  Full, ragged,
    one-key and empty key lists; `q_scale` 4 raises the softmax reference in later tiles (accumulators folded into
    registers); small and large cache scales; 4, 8 and 16 heads (one, two or four head groups).  Against the fp32 definition and
    against the mma.sync kernel through the switch."""
    from slopllm_b200.ops import native as N
    from slopllm_b200.ops import tcgen05
    cfg = mini_cfg(num_attention_heads=h, index_topk=2048)
    ops, ref = cuda_ops(cfg), RefOps(cfg)
    g = torch.Generator(device=DEV).manual_seed(900 + h + T)
    Rr, Dr, k = cfg.kv_lora_rank, cfg.qk_rope_head_dim, cfg.index_topk
    nslots = 4096
    cache = type("C", (), {})()
    lat = torch.randn(nslots, Rr, device=DEV, generator=g) * kv_scale
    lat[:, 128:256] *= 0.1                       # group scales of one row differ by an order of magnitude
    cache.kv = quant.pack_kv_rows(lat, torch.randn(nslots, Dr, device=DEV, generator=g), cfg.kv_quant_group)
    q_abs = (torch.randn(T, h, Rr, device=DEV, generator=g) * q_scale / max(kv_scale, 1.0)).to(torch.bfloat16)
    q_pe = (torch.randn(T, h, Dr, device=DEV, generator=g) * q_scale).to(torch.bfloat16)
    slots = torch.full((T, k), -1, dtype=torch.int32, device=DEV)
    lens = ([k, 1000, 0, 129, 128, 1, 127, 300] * (T // 8 + 1))[:T]
    lengths = torch.tensor(lens, dtype=torch.int32, device=DEV)
    for t in range(T):
        n = lens[t]
        slots[t, :n] = torch.randperm(nslots, device=DEV, generator=g)[:n].to(torch.int32)
    assert ops._mla_splits(T, h) == 1
    launches = N.kernel_count()
    o, lse = ops.sparse_mla(q_abs, q_pe, cache, slots, lengths)
    assert N.kernel_count() == launches + 1
    tcgen05.check_errors(torch.device(DEV))
    eo, elo = ref.sparse_mla(q_abs, q_pe, cache, slots, lengths)
    live = lengths > 0
    close(o, eo, what="sparse mla o (tcgen05)")
    close(lse[live], elo[live], tol=2e-3, what="lse (tcgen05)")
    assert torch.isinf(lse[~live]).all() and (o[~live] == 0).all()
    N.kernels().sl_sparse_mla_set_tcgen05(0)
    try:
        o2, lse2 = ops.sparse_mla(q_abs, q_pe, cache, slots, lengths)
    finally:
        N.kernels().sl_sparse_mla_set_tcgen05(3)
    close(o, o2, what="tcgen05 vs mma.sync")
    close(lse[live], lse2[live], tol=2e-3, what="lse, tcgen05 vs mma.sync")


def test_sparse_mla_on_tcgen05_keeps_a_long_tail_of_small_weights():
    """One key takes about 90 % of the softmax mass and two thousand keys share the rest at about 5e-5 each: the
    two-term e4m3 probabilities must still carry that tail (their common value component is visible in the output)."""
    from slopllm_b200.ops import tcgen05
    h, T = 8, 160
    cfg = mini_cfg(num_attention_heads=h, index_topk=2048)
    ops, ref = cuda_ops(cfg), RefOps(cfg)
    g = torch.Generator(device=DEV).manual_seed(4242)
    Rr, Dr, k = cfg.kv_lora_rank, cfg.qk_rope_head_dim, cfg.index_topk
    nslots = 4096
    lat = torch.zeros(nslots, Rr, device=DEV)
    lat[:, :Rr // 2] = torch.randn(nslots, Rr // 2, device=DEV, generator=g)
    lat[:, Rr // 2:] = 1.0                                   # the tail's common value component
    heavy = torch.arange(T, device=DEV)                     # token t's dominant key is slot t
    lat[heavy, Rr // 2:] = 0.0
    cache = type("C", (), {})()
    cache.kv = quant.pack_kv_rows(lat, torch.zeros(nslots, Dr, device=DEV), cfg.kv_quant_group)
    deq, _ = quant.unpack_kv_rows(cache.kv, Rr, Dr, cfg.kv_quant_group)
    k0 = deq[heavy]                                          # [T, R]
    alpha = 10.0 / ((k0 * k0).sum(-1, keepdim=True) * cfg.softmax_scale)
    q_abs = (alpha * k0)[:, None, :].expand(T, h, Rr).contiguous().to(torch.bfloat16)
    q_pe = torch.zeros(T, h, Dr, device=DEV, dtype=torch.bfloat16)
    slots = torch.empty(T, k, dtype=torch.int32, device=DEV)
    for t in range(T):
        others = torch.randperm(nslots - T, device=DEV, generator=g)[:k - 1] + T
        slots[t] = torch.cat([others[:1000], heavy[t:t + 1], others[1000:]]).to(torch.int32)    # the dominant key sits in a middle tile
    lengths = torch.full((T,), k, dtype=torch.int32, device=DEV)
    assert ops._mla_splits(T, h) == 1
    o, lse = ops.sparse_mla(q_abs, q_pe, cache, slots, lengths)
    tcgen05.check_errors(torch.device(DEV))
    eo, elo = ref.sparse_mla(q_abs, q_pe, cache, slots, lengths)
    tail = eo[:, :, Rr // 2:].float().mean().item()
    assert 0.02 < tail < 0.3, tail                           # the scenario is what the docstring says
    close(o, eo, what="sparse mla o with a long tail")
    rel = ((o[:, :, Rr // 2:].float().mean() - tail).abs() / tail).item()
    assert rel < 0.02, rel
    close(lse, elo, tol=2e-3, what="lse with a long tail")


@pytest.mark.parametrize("T,h", [(1, 8), (3, 8), (8, 8), (13, 4), (32, 8)])
def test_attention_output_merge_fused_with_value_expansion(T, h):
    """Decode attention output in one launch (merge of the key splits as the staging step of the value expansion, plus
    the fragment-ordered copy for the output projection) equals merge kernel + product + staging kernel bit for bit,
    and the fp32 definition within rounding."""
    from slopllm_b200.ops import native as N
    cfg = mini_cfg(num_attention_heads=h, index_topk=2048)
    ops, ref = cuda_ops(cfg), RefOps(cfg)
    g = torch.Generator(device=DEV).manual_seed(7 * T + h)
    Rr, Dr, k, Dv = cfg.kv_lora_rank, cfg.qk_rope_head_dim, cfg.index_topk, cfg.v_head_dim
    nslots = 4096
    cache = type("C", (), {})()
    cache.kv = quant.pack_kv_rows(torch.randn(nslots, Rr, device=DEV, generator=g), torch.randn(nslots, Dr, device=DEV, generator=g),
                                  cfg.kv_quant_group)
    q_abs = (torch.randn(T, h, Rr, device=DEV, generator=g) * 0.5).to(torch.bfloat16)
    q_pe = (torch.randn(T, h, Dr, device=DEV, generator=g) * 0.5).to(torch.bfloat16)
    slots = torch.full((T, k), -1, dtype=torch.int32, device=DEV)
    lens = ([k, 70, 0, 1, 1500] * 8)[:T]
    lengths = torch.tensor(lens, dtype=torch.int32, device=DEV)
    for t in range(T):
        slots[t, :lens[t]] = torch.randperm(nslots, device=DEV, generator=g)[:lens[t]].to(torch.int32)
    w_v = (torch.randn(h, Rr, Dv, device=DEV, generator=g) * 0.05).to(torch.bfloat16)
    assert ops._mla_splits(T, h) > 1
    fused = ops.attn_values(q_abs, q_pe, cache, slots, lengths, w_v)
    o, _ = ops.sparse_mla(q_abs, q_pe, cache, slots, lengths)
    plain = ops.v_expand(o, w_v)
    assert torch.equal(fused, plain)
    eo, _ = ref.sparse_mla(q_abs, q_pe, cache, slots, lengths)
    close(fused, ref.v_expand(eo, w_v), what="attention values")
    if T >= 2:
        K = h * Dv
        tpad = (T + 7) // 8 * 8
        want = torch.empty(tpad * K, dtype=torch.float16, device=DEV)
        N.call("sl_permute_x", want.data_ptr(), plain.data_ptr(), T, K, plain.stride(0), N.stream())
        assert torch.equal(fused._sl_perm, want)
    else:
        assert getattr(fused, "_sl_perm", None) is None


@pytest.mark.parametrize("T", [1, 4, 9])
def test_moe_small_and_dense(T):
    cfg = mini_cfg(hidden_size=2048, moe_intermediate_size=512)
    ops, ref = cuda_ops(cfg), RefOps(cfg)
    lw = random_layer(cfg, 1, 0, DEV, torch.bfloat16)
    g = torch.Generator(device=DEV).manual_seed(T)
    x = torch.randn(T, cfg.hidden_size, device=DEV, generator=g).to(torch.bfloat16)
    close(ops.moe_tp(x, lw), ref.moe_tp(x, lw), tol=2e-2, what="moe_tp")
    lw0 = random_layer(cfg, 0, 0, DEV, torch.bfloat16)
    close(ops.dense_mlp(x, lw0), ref.dense_mlp(x, lw0), tol=2e-2, what="dense mlp")


@pytest.mark.parametrize("T", [1, 8, 32])
def test_moe_fused_router_glm5_routing(T):
    """Router product + grouped sigmoid top-8 + plan in the first kernel of the layer (256 experts,
    8 groups) against the stand-alone route kernel followed by the same expert kernels."""
    cfg = mini_cfg(hidden_size=1024, moe_intermediate_size=256, n_routed_experts=256, num_experts_per_tok=8, n_group=8,
                   topk_group=4)
    ops, ref = cuda_ops(cfg), RefOps(cfg)
    ops._fp4_decode_force = "0"                       # this test pins the weight-streaming path (16-bit activations)
    lw = random_layer(cfg, 1, 0, DEV, torch.bfloat16)
    x = torch.randn(T, cfg.hidden_size, device=DEV, generator=torch.Generator(device=DEV).manual_seed(T)).to(torch.bfloat16)
    fused = ops.moe_tp(x, lw)
    ids, wts = ops.route(x, lw)
    unfused = ops._moe_small(x, lw.experts, lw.shared, ids, wts)
    close(fused, unfused, tol=2e-3, what="fused vs unfused router")
    close(fused, ref.moe_tp(x, lw), tol=2e-2, what="fused router vs reference")
    # the kernels must leave their counters at zero for the next call
    assert int(ops._zero_counter(x.device).item()) == 0
    assert int(ops._persist_sync(x.device).abs().sum().item()) == 0
    close(ops.moe_tp(x, lw), fused, tol=1e-6, what="second call")


@pytest.mark.parametrize("T,H,E,k", [(32, 2048, 64, 12), (30, 6144, 32, 16), (7, 7168, 128, 6), (20, 1024, 38, 4)])
def test_moe_router_plan_shapes(T, H, E, k):
    """The fused router kernel beyond the production shape: more than 256 routes (the plan takes several passes), more
    K steps than a warp keeps in registers, an expert count that leaves the last block partly empty, few experts with
    many routes each (several chunks of 8 per expert)."""
    cfg = mini_cfg(hidden_size=H, moe_intermediate_size=128, n_routed_experts=E, num_experts_per_tok=k, n_group=1, topk_group=1)
    ops, ref = cuda_ops(cfg), RefOps(cfg)
    lw = random_layer(cfg, 1, 0, DEV, torch.bfloat16)
    x = torch.randn(T, H, device=DEV, generator=torch.Generator(device=DEV).manual_seed(T + E)).to(torch.bfloat16)
    fused = ops.moe_tp(x, lw)
    ids, wts = ops.route(x, lw)
    close(fused, ops._moe_small(x, lw.experts, lw.shared, ids, wts), tol=2e-3, what="fused vs unfused router")
    close(fused, ref.moe_tp(x, lw), tol=2e-2, what="fused router vs reference")
    assert int(ops._zero_counter(x.device).item()) == 0


@pytest.mark.parametrize("T,H,I,E,k,shared", [(8, 1024, 256, 16, 4, True), (32, 2048, 512, 64, 8, True), (2, 1024, 256, 8, 2, False),
                                              (19, 6144, 256, 256, 8, True), (32, 1024, 256, 8, 8, True)])
def test_moe_decode_on_fp4_gemms(T, H, I, E, k, shared, monkeypatch):
    """Decode-sized MoE on the block-scaled FP4 GEMMs (all tokens as the narrow operand of every expert tile, column-row
    tables instead of sort / gather, shared expert from a second weight set) against the fp32 definition with emulated
    4-bit activations, and against the weight-streaming path within the activation quantisation error."""
    from slopllm_b200.ops import gemm
    monkeypatch.setattr(gemm, "MOE_A4", True)
    cfg = mini_cfg(hidden_size=H, moe_intermediate_size=I, n_routed_experts=E, num_experts_per_tok=k, n_group=1, topk_group=1,
                   n_shared_experts=1 if shared else 0)
    ops, ref = cuda_ops(cfg), RefOps(cfg)
    lw = random_layer(cfg, 1, 0, DEV, torch.bfloat16)
    x = torch.randn(T, H, device=DEV, generator=torch.Generator(device=DEV).manual_seed(T + E)).to(torch.bfloat16)
    ids, wts = ops.route(x, lw)
    ops._fp4_decode_force = "1"
    assert ops._fp4_decode_ok(T, lw)
    got = ops._moe_fp4_decode(x, lw, ids, wts)
    from slopllm_b200.ops import tcgen05
    tcgen05.check_errors(DEV)
    stream = ops._moe_small(x, lw.experts, lw.shared, ids, wts)
    rel = float((got - stream).norm() / stream.norm())
    assert rel < 0.2, rel                                  # 4-bit activations against 16-bit ones
    want = R.moe_experts(x.float(), lw.experts, ids, wts, a4=True)
    if lw.shared is not None:
        want = want + R.moe_experts(x.float(), lw.shared, torch.zeros(T, 1, dtype=torch.int32, device=DEV),
                                    torch.ones(T, 1, device=DEV), a4=True)
    rel = float((got - want).norm() / want.norm())
    assert rel < 0.05, rel
    # through the public op, twice (the second call finds used scratch)
    a = ops.moe_tp(x, lw)
    b = ops.moe_tp(x, lw)
    assert torch.equal(a, b)
    close(a, got, tol=2e-3, what="public op (router in the fused kernel) vs given routes")


@pytest.mark.parametrize("T,H,I,E,k,ng,tg", [
    (1, 1024, 256, 256, 8, 8, 4), (8, 1024, 256, 256, 8, 8, 4), (32, 1024, 256, 256, 8, 8, 4),
    (5, 2048, 512, 16, 4, 4, 2), (19, 2048, 1024, 16, 4, 1, 1), (8, 3072, 128, 32, 4, 1, 1),
    (8, 6144, 256, 256, 8, 8, 4), (4, 6144, 2048, 32, 8, 1, 1)])
def test_moe_persistent_kernel_matches_five_launch_path(T, H, I, E, k, ng, tg):
    """The one-launch persistent MoE layer (tile queue + completion counters) against the five-launch path with the
    same arithmetic, against the fp32 reference, and twice in a row (its counters must be back at zero)."""
    cfg = mini_cfg(hidden_size=H, moe_intermediate_size=I, n_routed_experts=E, num_experts_per_tok=k, n_group=ng, topk_group=tg)
    ops, ref = cuda_ops(cfg), RefOps(cfg)
    ops._persist_moe = True
    ops._fp4_decode_force = "0"                       # both forms compared here keep 16-bit activations
    lw = random_layer(cfg, 1, 0, DEV, torch.bfloat16)
    x = torch.randn(T, H, device=DEV, generator=torch.Generator(device=DEV).manual_seed(T)).to(torch.bfloat16)
    fused = ops.moe_tp(x, lw)
    torch.cuda.synchronize()
    ops.check_persistent_status()
    sync = ops._persist_sync(x.device)
    assert int(sync.abs().sum().item()) == 0, sync[:16].tolist()
    ops._persist_moe = False
    old = ops.moe_tp(x, lw)
    ops._persist_moe = True
    close(fused, old, tol=2e-3, what="persistent vs five-launch")
    close(fused, ref.moe_tp(x, lw), tol=2e-2, what="persistent vs reference")
    close(ops.moe_tp(x, lw), fused, tol=1e-6, what="second call")
    # given routes (no router stage): the form that expert parallelism and the small-batch path call
    ids, wts = ops.route(x, lw)
    close(ops._moe_small(x, lw.experts, lw.shared, ids, wts), fused, tol=2e-3, what="given routes")
    ops.check_persistent_status()


@pytest.mark.parametrize("T", [1, 5, 8, 19])
def test_norm_emits_permuted_operand(T):
    """add+RMSNorm can write the permuted f16 operand of the NVFP4 tensor-core kernels itself: the linear and the
    MoE layer fed from it must give the same result as with their own permute launch."""
    cfg = mini_cfg(hidden_size=2048, moe_intermediate_size=512)
    ops = cuda_ops(cfg)
    lw = random_layer(cfg, 1, 0, DEV, torch.bfloat16)
    g = torch.Generator(device=DEV).manual_seed(T)
    x = torch.randn(T, cfg.hidden_size, device=DEV, generator=g)
    res = torch.randn(T, cfg.hidden_size, device=DEV, generator=g)
    plain, _ = ops.add_rmsnorm(x, res, lw.post_attn_norm)
    perm, _ = ops.add_rmsnorm(x, res, lw.post_attn_norm, want_perm=True)
    assert torch.equal(plain, perm) and getattr(perm, "_sl_perm", None) is not None
    w = LinearWeight(*quant.random_nvfp4((768, cfg.hidden_size), g, DEV))
    if T >= 2:
        assert torch.equal(ops.linear(perm, w, out_f32=True), ops.linear(plain, w, out_f32=True))
    close(ops.moe_tp(perm, lw), ops.moe_tp(plain, lw), tol=1e-6, what="moe with emitted operand")


def test_moe_large_matches_reference(monkeypatch):
    """Prefill-sized MoE.  With 16-bit activations (SLOPLLM_B200_MOE_A4=0: the expansion kernels) against the fp32
    reference; on the default block-scaled FP4 path against the reference with the same NVFP4 activation rows."""
    from slopllm_b200.ops import gemm
    cfg = mini_cfg(hidden_size=1024, moe_intermediate_size=256)
    ops, ref = cuda_ops(cfg), RefOps(cfg)
    lw = random_layer(cfg, 1, 0, DEV, torch.bfloat16)
    x = torch.randn(200, cfg.hidden_size, device=DEV, generator=torch.Generator(device=DEV).manual_seed(4)).to(torch.bfloat16)
    exact = ref.moe_tp(x, lw)
    monkeypatch.setattr(gemm, "MOE_A4", False)
    close(ops.moe_tp(x, lw), exact, tol=2e-2, what="moe large, 16-bit activations")
    monkeypatch.setattr(gemm, "MOE_A4", True)
    assert gemm.fp4_moe_ok(lw.experts, cfg.hidden_size)
    y4 = ops.moe_tp(x, lw)
    ids, w = ref.route(x, lw)
    T = x.shape[0]
    emul = R.moe_experts(x, lw.experts, ids, w, a4=True) + R.moe_experts(
        x, lw.shared, torch.zeros(T, 1, dtype=torch.int32, device=DEV), torch.ones(T, 1, device=DEV), a4=True)
    # re-quantising the activations is discontinuous (a value next to a rounding boundary may take either code), so the
    # emulation agrees in the mean, not element by element
    rel_emul = ((y4.float() - emul).norm() / emul.norm()).item()
    assert rel_emul < 0.05, rel_emul
    close(y4, exact, tol=0.25, what="moe large, NVFP4 activations vs 16-bit activations")
    rel = ((y4.float() - exact).norm() / exact.norm()).item()
    assert rel < 0.2, rel                    # two NVFP4 roundings of the activations (rows in, SiLU * mul out): ~0.1 each


@pytest.mark.parametrize("M,N,K", [(300, 512, 1024), (129, 200, 64), (4096, 768, 2048)])
@pytest.mark.parametrize("out_kind", [0, 1, 2])
def test_gemm_w4_fused_dequant(M, N, K, out_kind):
    """NVFP4-weight GEMM that expands the weight tile inside the kernel, against x @ dequant(W)^T in fp32
    (ragged M and N, one and two global scales, the three output types)."""
    from slopllm_b200.ops import gemm, tcgen05
    g = torch.Generator(device=DEV).manual_seed(M + N + K)
    wq, ws, _ = quant.random_nvfp4((N, K), g, DEV)
    x = torch.randn(M, K, device=DEV, generator=g).to(torch.bfloat16)
    for gs, split in ((torch.tensor([0.75], device=DEV), 0), (torch.tensor([0.5, 2.0], device=DEV), 128)):
        y = gemm.gemm_w4(gemm.to_f16_rows(x), wq, ws, gs, out_kind, split=split)
        wd = quant.nvfp4_dequantize(wq, ws, torch.ones((), device=DEV), torch.float32)
        col = torch.full((N,), float(gs[0]), device=DEV) if gs.numel() == 1 else torch.where(
            torch.arange(N, device=DEV) < split, gs[0], gs[1])
        ref = (x.float() @ wd.t()) * col
        assert y.dtype == {0: torch.bfloat16, 1: torch.float32, 2: torch.float16}[out_kind]
        close(y, ref, tol=1e-2, what=f"w4 gemm {M}x{N}x{K} kind={out_kind} scales={gs.numel()}")
    assert int(tcgen05.error_flag(x.device)[0]) == 0


def test_grouped_gemm_w4_ragged_groups():
    """Grouped NVFP4-weight GEMM over expert-sorted rows: empty groups, groups shorter and longer than a 128-row tile."""
    from slopllm_b200.ops import gemm, tcgen05
    g = torch.Generator(device=DEV).manual_seed(5)
    G, N, K = 6, 512, 256
    counts = [0, 130, 7, 0, 256, 91]
    M = sum(counts)
    wq, ws, _ = quant.random_nvfp4((G, N, K), g, DEV)
    gs = torch.rand(G, 2, device=DEV, generator=g) + 0.5
    a = torch.randn(M, K, device=DEV, generator=g).to(torch.bfloat16)
    off = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32, device=DEV)
    for bn in (128, 256):
        c = gemm.grouped_gemm_w4(gemm.to_f16_rows(a), wq, ws, gs, off, 1, split=N // 2, bn=bn)
        r0 = 0
        for gi, n in enumerate(counts):
            if n == 0:
                continue
            wd = quant.nvfp4_dequantize(wq[gi], ws[gi], torch.ones((), device=DEV), torch.float32)
            col = torch.where(torch.arange(N, device=DEV) < N // 2, gs[gi, 0], gs[gi, 1])
            close(c[r0:r0 + n], (a[r0:r0 + n].float() @ wd.t()) * col, tol=1e-2, what=f"grouped w4 group {gi} bn={bn}")
            r0 += n
    assert int(tcgen05.error_flag(a.device)[0]) == 0


@pytest.mark.parametrize("n_tok,k,E,offset", [(5, 4, 16, 0), (700, 8, 256, 0), (300, 8, 32, 64)])
def test_moe_sort_routes_matches_stable_sort(n_tok, k, E, offset):
    """Counting sort of routes by expert (prefill MoE) against a stable torch sort; `offset` makes some experts non-local."""
    from slopllm_b200.ops import native as N
    g = torch.Generator(device=DEV).manual_seed(n_tok)
    total_e = E + 2 * offset
    ids = torch.randint(0, total_e, (n_tok * k,), device=DEV, generator=g, dtype=torch.int32)
    M = ids.numel()
    scratch = torch.empty(((M + 1023) // 1024) * (E + 1), dtype=torch.int32, device=DEV)
    offsets = torch.empty(E + 1, dtype=torch.int32, device=DEV)
    order, rows_of, src_tok = (torch.empty(M, dtype=torch.int32, device=DEV) for _ in range(3))
    N.call("sl_moe_sort_routes", ids.data_ptr(), M, k, offset, E, scratch.data_ptr(), offsets.data_ptr(), order.data_ptr(),
           rows_of.data_ptr(), src_tok.data_ptr(), N.stream())
    local = ids.long() - offset
    key = torch.where((local >= 0) & (local < E), local, torch.full_like(local, E))
    exp_order = torch.argsort(key, stable=True)
    counts = torch.bincount(key, minlength=E + 1)
    exp_off = torch.cat([torch.zeros(1, dtype=torch.long, device=DEV), counts.cumsum(0)])[:E + 1]
    assert torch.equal(order.long(), exp_order)
    assert torch.equal(offsets.long(), exp_off)
    assert torch.equal(src_tok.long(), exp_order // k)
    inv = torch.empty_like(exp_order)
    inv[exp_order] = torch.arange(M, device=DEV)
    assert torch.equal(rows_of.long(), torch.where(key < E, inv, torch.full_like(inv, -1)))


def test_argmax():
    ops = cuda_ops(GlmMoeDsaConfig.tiny())
    x = torch.randn(5, 154880, device=DEV)
    assert torch.equal(ops.argmax(x), x.argmax(-1))
    assert torch.equal(ops.argmax(x.to(torch.bfloat16), id_offset=10), x.to(torch.bfloat16).float().argmax(-1) + 10)


_ = math
