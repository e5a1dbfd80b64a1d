"""Fused NVLink collectives.  Single GPU: W ranks are emulated as W regions on one device (every
producer runs before any consumer, so no kernel ever waits on another launch).  Two or more GPUs:
real peer memory, one process per GPU."""
import os
import socket

import pytest
import torch

from slopllm_b200.config import GlmMoeDsaConfig
from slopllm_b200.models.weights import LinearWeight, random_layer
from slopllm_b200.ops import RefOps, quant, reference as R

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _regions(W, rows, row_len, **kw):
    from slopllm_b200.parallel.nvlink import SymmetricRegion
    lay = SymmetricRegion.layout(W, rows, row_len, kw.get("gather_bytes", 0), kw.get("cp_shape"))
    bufs = [torch.zeros(lay["total"], dtype=torch.uint8, device=DEV) for _ in range(W)]
    ptrs = [b.data_ptr() for b in bufs]
    return [SymmetricRegion(r, W, rows, row_len, bufs[r], ptrs, **kw) for r in range(W)]


def _close(a, b, tol=1e-2):
    a, b = a.float(), b.float()
    assert ((a - b).abs().max() / b.abs().max().clamp(min=1e-6)).item() <= tol


@pytest.mark.parametrize("W", [2, 4, 8])
@pytest.mark.parametrize("T", [1, 5, 32])
def test_fused_allreduce_emulated_ranks(W, T):
    from slopllm_b200.ops.cuda_ops import CudaOps
    from slopllm_b200.parallel.dist import ParallelContext
    from slopllm_b200.parallel.nvlink import NvlinkComm, PushSink
    cfg = GlmMoeDsaConfig.tiny()
    H, K = 1024, 512
    ops = CudaOps(cfg)
    regions = _regions(W, 32, H)
    comms = [NvlinkComm(ParallelContext(r, W, torch.device(DEV)), cfg, region=regions[r]) for r in range(W)]
    g = torch.Generator(device=DEV).manual_seed(W * 100 + T)
    res = torch.randn(T, H, device=DEV, generator=g)
    norm_w = torch.rand(H, device=DEV, generator=g).to(torch.bfloat16)
    for rounds in range(3):            # three uses: exercises the epoch counters and buffer rotation
        xs = [torch.randn(T, K, device=DEV, generator=g).to(torch.bfloat16) for _ in range(W)]
        ws = [LinearWeight(*quant.random_nvfp4((H, K), g, DEV)) if rounds != 1 else
              LinearWeight((torch.randn(H, K, device=DEV, generator=g) * 0.05).to(torch.bfloat16)) for _ in range(W)]
        sinks = []
        for r in range(W):
            comms[r].begin_forward()
            sinks.append(ops.linear(xs[r], ws[r], out_f32=True, sink=comms[r].partial_sink(T)))
        expect = sum(R.linear(xs[r], ws[r]) for r in range(W))
        eo, er = R.add_rmsnorm(expect, res, norm_w, 1e-5)
        for r in range(W):
            assert isinstance(sinks[r], PushSink)
            out, newres = comms[r].allreduce_add_rmsnorm(ops, sinks[r], res, norm_w, 1e-5)
            _close(newres, er)
            _close(out, eo)
            comms[r].check_status()
    from slopllm_b200.ops import tcgen05
    torch.cuda.synchronize()
    tcgen05.check_errors(DEV)
    for rg in regions:                 # no producer stored past the end of a receive slot
        rg.check_canaries()


def test_moe_down_push_emulated():
    from slopllm_b200.ops.cuda_ops import CudaOps
    from slopllm_b200.parallel.dist import ParallelContext
    from slopllm_b200.parallel.nvlink import NvlinkComm
    W, T = 2, 3
    cfg = GlmMoeDsaConfig(hidden_size=1024, moe_intermediate_size=512, num_hidden_layers=2, num_attention_heads=8,
                          q_lora_rank=256, n_routed_experts=16, num_experts_per_tok=4, n_group=4, topk_group=2,
                          first_k_dense_replace=1, vocab_size=1024)
    ops, ref = CudaOps(cfg), RefOps(cfg)
    regions = _regions(W, 32, cfg.hidden_size)
    comms = [NvlinkComm(ParallelContext(r, W, torch.device(DEV)), cfg, region=regions[r]) for r in range(W)]
    lws = [random_layer(cfg, 1, 0, DEV, torch.bfloat16, tp_rank=r, tp_world=W) for r in range(W)]
    x = torch.randn(T, cfg.hidden_size, device=DEV, generator=torch.Generator(device=DEV).manual_seed(4)).to(torch.bfloat16)
    res = torch.zeros(T, cfg.hidden_size, device=DEV)
    ones = torch.ones(cfg.hidden_size, device=DEV, dtype=torch.bfloat16)
    sinks = []
    for r in range(W):
        comms[r].begin_forward()
        sinks.append(ops.moe_tp(x, lws[r], sink=comms[r].partial_sink(T)))
    expect = sum(ref.moe_tp(x, lws[r]) for r in range(W))
    for r in range(W):
        _, total = comms[r].allreduce_add_rmsnorm(ops, sinks[r], res, ones, 1e-5)
        _close(total, expect, 2e-2)


def test_wait_times_out_cleanly():
    """A flag that nothing sets: the kernel gives up after its spin budget, records the site and
    returns; the context stays usable."""
    from slopllm_b200.ops import native as N
    from slopllm_b200.parallel.nvlink import CollectiveTimeout
    region = _regions(2, 8, 256)[0]
    region.wait_spins = 2000
    flag = torch.zeros(4, dtype=torch.int32, device=DEV)
    N.call("sl_wait_flag", flag.data_ptr(), 5, 2000, region.status_ptr, N.stream())
    torch.cuda.synchronize()
    with pytest.raises(CollectiveTimeout):
        region.check_status()
    region.check_status()                          # cleared
    assert float((torch.ones(4, device=DEV) * 2).sum()) == 8.0


def test_tagged_consumer_times_out_cleanly():
    """The all-reduce consumer polls tagged words; when no producer ever writes them it gives up after
    its poll budget, records the timeout in the status block and finishes, leaving the context usable."""
    import ctypes as C
    from slopllm_b200.ops import native as N
    from slopllm_b200.parallel.nvlink import CollectiveTimeout
    H, T = 256, 2
    region = _regions(2, 8, H, wait_spins=300)[0]
    out = torch.empty(T, H, dtype=torch.bfloat16, device=DEV)
    res = torch.empty(T, H, dtype=torch.float32, device=DEV)
    w = torch.ones(H, dtype=torch.bfloat16, device=DEV)
    N.call("sl_ar_add_rmsnorm", C.byref(region.recv_ctx[0]), out.data_ptr(), res.data_ptr(), 0, w.data_ptr(), T, H, 1e-5, 0, N.stream())
    torch.cuda.synchronize()
    with pytest.raises(CollectiveTimeout):
        region.check_status()
    region.check_status()
    assert float((torch.ones(4, device=DEV) * 2).sum()) == 8.0


def test_cp_merge_push_emulated():
    from slopllm_b200.ops.cuda_ops import CudaOps
    from slopllm_b200.parallel.dist import ParallelContext
    from slopllm_b200.parallel.nvlink import NvlinkComm
    W, T, h, Rr, S = 4, 3, 8, 512, 5
    cfg = GlmMoeDsaConfig(hidden_size=1024, num_attention_heads=h, num_hidden_layers=1, vocab_size=1024)
    ops = CudaOps(cfg)
    regions = _regions(W, 32, cfg.hidden_size, cp_shape=(32, h, Rr))
    comms = [NvlinkComm(ParallelContext(r, W, torch.device(DEV), cp=True), cfg, region=regions[r]) for r in range(W)]
    g = torch.Generator(device=DEV).manual_seed(9)
    o_parts = [torch.randn(T, h, S, Rr, device=DEV, generator=g) for _ in range(W)]
    l_parts = [torch.randn(T, h, S, device=DEV, generator=g) * 3 for _ in range(W)]
    l_parts[1][0, 2, :] = float("-inf")            # a rank with no visible key for one (token, head)
    # emulate: every rank pushes, then every rank merges
    from slopllm_b200.ops import native as N
    import ctypes as C
    hl = h // W
    for rnd in range(3):                     # three merges in a row: the staging halves alternate with the epoch parity
        staged = []
        for r in range(W):
            o, lse = ops.combine_f32([o_parts[r] * (rnd + 1)], [l_parts[r]])
            staged.append((o, lse))
            N.call("sl_cp_merge_push", C.byref(regions[r].cp_ctx), o.data_ptr(), lse.data_ptr(), T, N.stream())
        allo = torch.stack([s[0] for s in staged])
        alll = torch.stack([s[1] for s in staged])
        expect, _ = R.merge_attention_partials(allo, alll)
        for r in range(W):
            rg = regions[r]
            N.call("sl_epoch_wait", rg.peer_ptrs[r] + rg.lay["flags"][4], rg.state.data_ptr() + 16, W, rg.wait_spins,
                   rg.status_ptr, 5, N.stream())
            so = rg.local_view(rg.lay["cp_o"], W * 32 * hl * Rr * 4).view(torch.float32).view(W, 32, hl, 1, Rr)
            sl = rg.local_view(rg.lay["cp_lse"], W * 32 * hl * 4).view(torch.float32).view(W, 32, hl, 1)
            merged, _ = ops.combine([so[i] for i in range(W)], [sl[i] for i in range(W)], rows=T, want_lse=False,
                                    parity=(rg.state.data_ptr() + 16, W * 32 * hl * Rr, W * 32 * hl))
            _close(merged, expect[:, r * hl:(r + 1) * hl])
            rg.check_status()


# ---- real multi-GPU -------------------------------------------------------------------------------


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _mgpu_worker(rank, world, port, q, cp=False, bulk=False):
    import dataclasses
    import traceback
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    if bulk:        # prefill chunks of 64 rows (32 per rank) take the reduce-scatter / all-gather kernels
        os.environ["SLOPLLM_B200_BULK_AR"] = "1"
    try:
        import torch.distributed as dist
        from slopllm_b200.models.glm_moe_dsa import GlmMoeDsaModel
        from slopllm_b200.models.weights import random_model
        from slopllm_b200.parallel.dist import init_from_env
        from slopllm_b200.parallel.fused import make_comm
        from slopllm_b200.runtime.engine import Engine
        ctx = init_from_env()
        if cp:
            ctx = dataclasses.replace(ctx, cp=True)      # KV tokens interleaved over the ranks, weights stay TP-sharded
        cfg = GlmMoeDsaConfig(hidden_size=1024, intermediate_size=2048, moe_intermediate_size=512, num_hidden_layers=3,
                              num_nextn_predict_layers=0, vocab_size=2048, num_attention_heads=8, q_lora_rank=256,
                              n_routed_experts=16, num_experts_per_tok=4, n_group=4, topk_group=2, index_topk=64,
                              first_k_dense_replace=1, quant_o_proj=True, quant_dense_mlp=True)
        w = random_model(cfg, 0, ctx.device, torch.bfloat16, ctx.rank, ctx.world, with_mtp=False)
        g = torch.Generator().manual_seed(1)
        prompts = [torch.randint(0, cfg.vocab_size, (100,), generator=g).tolist() for _ in range(2)]
        out = {}
        for fused in (False, True):
            comm = make_comm(ctx, cfg, fused=fused)
            eng = Engine(cfg, GlmMoeDsaModel(cfg, w, ctx, comm=comm), num_pages=16, max_batch=2, max_seq_len=512)
            seqs = [eng.kv.new_sequence() for _ in range(2)]
            last, _ = eng.prefill(seqs, prompts, chunk_size=64)
            toks = [list(last)]
            for _ in range(6):
                last = eng.decode_step(seqs, last)
                toks.append(list(last))
            comm.check_status()
            out[fused] = toks
        dist.barrier()
        torch.cuda.synchronize()
        q.put((rank, out, None))
    except Exception:  # noqa: BLE001
        q.put((rank, None, traceback.format_exc()))
    # leave without tearing down NCCL communicators that captured graphs still reference
    q.close()
    q.join_thread()
    os._exit(0)


@pytest.mark.multigpu
@pytest.mark.parametrize("cp,bulk", [(False, False), (True, False), (False, True)])
def test_tp2_fused_equals_nccl_on_two_gpus(cp, bulk):
    """Prefill + graph-captured decode on two GPUs, in-kernel NVLink collectives against NCCL; with `cp` the KV is
    sharded by token and the indexer top-k / attention partials are merged across the ranks; with `bulk` the prefill
    chunks' all-reduces run as reduce-scatter from the GEMM epilogue + all-gather over peer memory."""
    import torch.multiprocessing as mp
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_mgpu_worker, args=(r, world, port, q, cp, bulk), daemon=True) for r in range(world)]
    for p in procs:
        p.start()
    res = {}
    try:
        for _ in range(world):
            rank, out, err = q.get(timeout=300)
            assert err is None, err
            res[rank] = out
    finally:
        for p in procs:
            p.join(timeout=20)
            if p.is_alive():
                p.kill()
    assert res[0] == res[1]
    if bulk:
        # the bulk path rounds partial sums to bf16 on the wire, so a near-tie of random-init logits may resolve differently
        # from the fp32 library sum: the ranks must agree with each other (above) and no wait may have expired (the worker
        # checks); the numerics are pinned by the emulated-rank test against the fp32 definition
        return
    # fused and library collectives sum in different orders: allow a late near-tie flip
    assert res[0][True][:4] == res[0][False][:4]


def _ep_worker(rank, world, port, q):
    """Expert parallelism on real GPUs: prefill chunks of 64 rows take the peer-memory dispatch / combine kernels
    (`parallel/ep.py`); the same run with that path switched off (every rank computes its experts for all rows and the
    all-reduce sums) must produce the same tokens."""
    import traceback
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    try:
        import torch.distributed as dist
        from slopllm_b200.models.glm_moe_dsa import GlmMoeDsaModel
        from slopllm_b200.models.weights import random_model
        from slopllm_b200.parallel.dist import init_from_env
        from slopllm_b200.parallel.fused import make_comm
        from slopllm_b200.runtime.engine import Engine
        ctx = init_from_env(ep=True)
        cfg = GlmMoeDsaConfig(hidden_size=1024, intermediate_size=2048, moe_intermediate_size=512, num_hidden_layers=3,
                              num_nextn_predict_layers=0, vocab_size=2048, num_attention_heads=8, q_lora_rank=256,
                              n_routed_experts=16, num_experts_per_tok=4, n_group=4, topk_group=2, index_topk=64,
                              first_k_dense_replace=1, quant_o_proj=True, quant_dense_mlp=True)
        w = random_model(cfg, 0, ctx.device, torch.bfloat16, ctx.rank, ctx.world, ep=True, with_mtp=False)
        g = torch.Generator().manual_seed(1)
        prompts = [torch.randint(0, cfg.vocab_size, (100,), generator=g).tolist() for _ in range(2)]
        out = {}
        for fused_ep in (False, True):
            comm = make_comm(ctx, cfg, fused=True)
            model = GlmMoeDsaModel(cfg, w, ctx, comm=comm)
            model._ep_unavailable = not fused_ep
            eng = Engine(cfg, model, num_pages=16, max_batch=2, max_seq_len=512)
            seqs = [eng.kv.new_sequence() for _ in range(2)]
            last, _ = eng.prefill(seqs, prompts, chunk_size=64)
            toks = [list(last)]
            for _ in range(4):
                last = eng.decode_step(seqs, last)
                toks.append(list(last))
            comm.check_status()
            if fused_ep:
                assert model._ep_exchange is not None
                model._ep_exchange.check_status()
                out["rounds"] = int(model._ep_exchange.state[0])
            out[fused_ep] = toks
        dist.barrier()
        torch.cuda.synchronize()
        q.put((rank, out, None))
    except Exception:  # noqa: BLE001
        q.put((rank, None, traceback.format_exc()))
    q.close()
    q.join_thread()
    os._exit(0)


@pytest.mark.multigpu
def test_ep_dispatch_combine_on_two_gpus():
    import torch.multiprocessing as mp
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_ep_worker, args=(r, world, port, q), daemon=True) for r in range(world)]
    for p in procs:
        p.start()
    res = {}
    try:
        for _ in range(world):
            rank, out, err = q.get(timeout=300)
            assert err is None, err
            res[rank] = out
    finally:
        for p in procs:
            p.join(timeout=20)
            if p.is_alive():
                p.kill()
    assert res[0] == res[1]                               # the ranks agree on every token
    # the two 100-token prompts are packed into chunks of 64, 64, 64 and 8 rows: the three full chunks of each of the
    # 2 MoE layers went through the exchange, the 8-row tail takes the small-batch path
    assert res[0]["rounds"] == 2 * 3
    # the home rank quantises a row exactly as every rank does on the other path: same tokens (allow a late near-tie)
    assert res[0][True][:3] == res[0][False][:3]
