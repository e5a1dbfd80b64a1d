"""Prefill-sized all-reduce as reduce-scatter (inside the GEMM epilogue) + all-gather + residual add + RMSNorm.
W ranks are emulated as W regions on one device and run phase by phase (all producers, then all owner steps, then
all consumers), so no kernel ever waits on a later launch."""
import pytest
import torch

from slopllm_b200.config import GlmMoeDsaConfig
from slopllm_b200.models.weights import LinearWeight
from slopllm_b200.ops import quant, reference as R

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _regions(W, row_len, bulk_rows):
    from slopllm_b200.parallel.nvlink import SymmetricRegion
    lay = SymmetricRegion.layout(W, 32, row_len, 0, None, bulk_rows)
    bufs = [torch.zeros(lay["total"], dtype=torch.uint8, device=DEV) for _ in range(W)]
    ptrs = [b.data_ptr() for b in bufs]
    return [SymmetricRegion(r, W, 32, row_len, bufs[r], ptrs, bulk_rows=bulk_rows) for r in range(W)]


def _close(a, b, tol=1e-2):
    a, b = a.float(), b.float()
    assert ((a - b).abs().max() / b.abs().max().clamp(min=1e-6)).item() <= tol


def _comms(W, H, bulk_rows):
    from slopllm_b200.parallel.dist import ParallelContext
    from slopllm_b200.parallel.nvlink import NvlinkComm
    cfg = GlmMoeDsaConfig.tiny()
    regions = _regions(W, H, bulk_rows)
    for rg in regions:
        rg.wait_spins = 200_000        # a broken protocol shows up as a recorded timeout within tens of milliseconds
    return cfg, [NvlinkComm(ParallelContext(r, W, torch.device(DEV)), cfg, region=regions[r]) for r in range(W)]


@pytest.mark.parametrize("W,T", [(2, 256), (4, 512), (8, 256), (2, 1024)])   # the last: more rows than resident waiting blocks
def test_bulk_allreduce_emulated_ranks(W, T):
    from slopllm_b200.ops import tcgen05
    from slopllm_b200.ops.cuda_ops import CudaOps
    from slopllm_b200.parallel.nvlink import BulkSink
    H, K = 1024, 512
    cfg, comms = _comms(W, H, max(512, T))
    ops = CudaOps(cfg)
    g = torch.Generator(device=DEV).manual_seed(W * 1000 + T)
    norm_w = torch.rand(H, device=DEV, generator=g).to(torch.bfloat16)
    # use 0: bf16 weights, GEMM epilogue is the producer; use 1: NVFP4 weights (expanded, same epilogue), no residual;
    # use 2: an existing fp32 tensor is pushed.  Three uses of the same lane also exercise the counter resets.
    for rnd in range(3):
        res = torch.randn(T, H, device=DEV, generator=g) if rnd != 1 else None
        xs = [torch.randn(T, K, device=DEV, generator=g).to(torch.bfloat16) for _ in range(W)]
        ws = [LinearWeight(*quant.random_nvfp4((H, K), g, DEV)) if rnd == 1 else
              LinearWeight((torch.randn(H, K, device=DEV, generator=g) * 0.05).to(torch.bfloat16)) for _ in range(W)]
        partials = [R.linear(xs[r], ws[r]) for r in range(W)]
        sinks = []
        for r in range(W):
            sink = comms[r].partial_sink(T)
            assert isinstance(sink, BulkSink) and sink.lane == 0
            if rnd == 2:
                sinks.append(sink.push_tensor(partials[r].to(torch.float32)))
            else:
                sinks.append(ops.linear(xs[r], ws[r], out_f32=True, sink=sink))
        for r in range(W):
            comms[r].bulk_reduce(sinks[r])
        expect = sum(partials)
        eo, er = R.add_rmsnorm(expect, res, norm_w, 1e-5)
        for r in range(W):
            out, newres = comms[r].bulk_finish(sinks[r], res, norm_w, 1e-5)
            _close(newres, er)
            _close(out, eo)
            comms[r].check_status()
    torch.cuda.synchronize()
    tcgen05.check_errors(DEV)
    for c in comms:      # nothing was stored past the end of an area; every arrival counter is back at zero
        c.region.check_canaries()
        assert int(c.region.bulk_state.abs().sum()) == 0
        lane = c.region.lay["bulk"][0]
        assert int(c.region.local_view(lane["rs_count"], 4 * 16).view(torch.int32).abs().sum()) == 0
        assert int(c.region.local_view(lane["ag_count"], 4 * 8).view(torch.int32).abs().sum()) == 0


def test_bulk_sink_falls_back():
    """Row counts the bulk path does not take (not a multiple of 32 rows per rank, larger than the lane) give no sink,
    so the caller keeps the library all-reduce."""
    _, comms = _comms(2, 1024, 512)
    assert comms[0].partial_sink(100) is None
    assert comms[0].partial_sink(1024) is None
    assert comms[0].partial_sink(128) is not None


def test_bulk_owner_wait_times_out_cleanly():
    """No producer ever delivers: the owner step gives up after its poll budget, records the timeout and returns;
    the context stays usable."""
    from slopllm_b200.parallel.nvlink import CollectiveTimeout
    _, comms = _comms(2, 256, 64)
    comms[0].region.wait_spins = 2000
    sink = comms[0].partial_sink(64)
    comms[0].bulk_reduce(sink)
    torch.cuda.synchronize()
    with pytest.raises(CollectiveTimeout):
        comms[0].check_status()
    assert float((torch.ones(4, device=DEV) * 2).sum()) == 8.0
