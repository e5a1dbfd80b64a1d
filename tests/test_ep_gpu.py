"""Expert-parallel dispatch / grouped FP4 GEMMs / combine over peer memory.  W ranks are emulated as W symmetric buffers on
one device and run phase by phase (all count pushes, then all dispatches, then all owners, then all combines), so no
kernel ever waits on a later launch."""
import pytest
import torch

from slopllm_b200.config import GlmMoeDsaConfig
from slopllm_b200.models.weights import random_layer
from slopllm_b200.ops import reference as R

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _cfg():
    return GlmMoeDsaConfig(hidden_size=1024, intermediate_size=1024, moe_intermediate_size=256, num_hidden_layers=2,
                           num_nextn_predict_layers=0, vocab_size=4096, num_attention_heads=8, q_lora_rank=512, kv_lora_rank=512,
                           qk_nope_head_dim=192, qk_rope_head_dim=64, v_head_dim=256, n_routed_experts=16, n_shared_experts=0,
                           num_experts_per_tok=4, n_group=1, topk_group=1, index_topk=256, index_head_dim=128, index_n_heads=32,
                           first_k_dense_replace=1)


def _close(a, b, tol, what):
    a, b = a.float(), b.float()
    err = ((a - b).abs().max() / b.abs().max().clamp(min=1e-6)).item()
    assert err <= tol, f"{what}: {err:.4g} > {tol}"


@pytest.mark.parametrize("W,T_total,cap_rows", [(4, 96, 0), (8, 40, 0), (2, 70, 0)])
def test_ep_round_matches_single_rank_fp4_path(W, T_total, cap_rows):
    from slopllm_b200.ops import tcgen05
    from slopllm_b200.ops.cuda_ops import CudaOps
    from slopllm_b200.parallel.ep import EpExchange
    cfg = _cfg()
    E, H, k = cfg.n_routed_experts, cfg.hidden_size, cfg.num_experts_per_tok
    ops = CudaOps(cfg)
    lw = random_layer(cfg, 1, 0, DEV, torch.bfloat16)
    slices = [lw.experts.ep_slice(r, W) for r in range(W)]
    per = -(-T_total // W)
    recv = cap_rows or T_total * k
    lay = EpExchange.layout(W, E, H, k, per, recv, 128)
    bufs = [torch.zeros(lay["total"], dtype=torch.uint8, device=DEV) for _ in range(W)]
    ptrs = [b.data_ptr() for b in bufs]
    exs = [EpExchange(r, W, E, H, k, per, recv, bufs[r], ptrs, 128, wait_spins=200_000) for r in range(W)]
    g = torch.Generator(device=DEV).manual_seed(W * 100 + T_total)
    for rnd in range(2):                                  # two rounds on the same buffers: the epoch tags must move on
        x = torch.randn(T_total, H, device=DEV, generator=g).to(torch.bfloat16)
        ids, wts = ops.route(x, lw)
        home = [(min(T_total, r * per), min(T_total, (r + 1) * per)) for r in range(W)]
        for r, (a, b) in enumerate(home):
            exs[r].route_and_count(ids[a:b])
        for r, (a, b) in enumerate(home):
            exs[r].plan_and_dispatch(x[a:b])
        for r in range(W):
            exs[r].experts(slices[r])
        outs = []
        for r, (a, b) in enumerate(home):
            outs.append(exs[r].combine(torch.zeros(b - a, H, device=DEV), wts[a:b]))
        torch.cuda.synchronize()
        for ex in exs:
            ex.check_status()
        tcgen05.check_errors(DEV)
        got = torch.cat(outs)
        # the same W4A4 arithmetic on one rank with all experts, and its PyTorch emulation
        one = ops.moe_local_experts(x, lw.experts, ids, wts)
        _close(got, one, 5e-3, f"round {rnd}: EP vs single-rank FP4 path")
        # re-quantising the activations is discontinuous: a PyTorch emulation agrees in the mean, not element by element
        emul = R.moe_experts(x, lw.experts, ids, wts, a4=True)
        rel = ((got - emul).norm() / emul.norm()).item()
        assert rel < 0.05, f"round {rnd}: EP vs emulation, relative L2 error {rel:.4g}"
    assert all(int(ex.state[0]) == 2 and int(ex.state[1]) == 0 for ex in exs)      # two rounds closed, tickets back at zero


def test_ep_wait_times_out_cleanly():
    """Nobody pushes counts: the plan kernel's wait runs out, records it and returns; the context stays usable."""
    from slopllm_b200.ops.native import CollectiveTimeout
    from slopllm_b200.parallel.ep import EpExchange
    cfg = _cfg()
    lay = EpExchange.layout(2, 16, 1024, 4, 8, 64, 128)
    bufs = [torch.zeros(lay["total"], dtype=torch.uint8, device=DEV) for _ in range(2)]
    ex = EpExchange(0, 2, 16, 1024, 4, 8, 64, bufs[0], [b.data_ptr() for b in bufs], 128, wait_spins=2000)
    ids = torch.zeros(4, 4, dtype=torch.int32, device=DEV)
    ex.route_and_count(ids)                               # rank 1 never does
    ex._order = torch.zeros(16, dtype=torch.int32, device=DEV)
    x = torch.zeros(4, 1024, dtype=torch.bfloat16, device=DEV)
    ex.plan_and_dispatch(x)
    torch.cuda.synchronize()
    with pytest.raises(CollectiveTimeout):
        ex.check_status()
    assert float((torch.ones(4, device=DEV) * 2).sum()) == 8.0
