"""Block-scaled NVFP4 tensor-core path (`tcgen05.mma.kind::mxf4nvf4`): scale-tile layout, activation quantiser, plain and
grouped products against fp32 PyTorch references of the same (quantised) operands."""
import pytest
import torch

from slopllm_b200.ops import quant

pytestmark = pytest.mark.gpu
DEV = "cuda"


def close(a, b, tol, what=""):
    a, b = a.to(torch.float32), b.to(torch.float32)
    assert a.shape == b.shape, (what, a.shape, b.shape)
    scale = b.abs().max().clamp(min=1e-6)
    err = ((a - b).abs().max() / scale).item()
    assert err <= tol, f"{what}: max rel-to-peak error {err:.4g} > {tol}"


def deq_rows(q, sf, g, bn=128):
    """fp32 value of quantised (ungrouped) activation rows: codes, scale tiles for GEMM tiles of `bn` rows, global scales."""
    from slopllm_b200.ops import fp4
    rows, K = q.shape[0], q.shape[1] * 2
    return quant.nvfp4_dequantize(q, fp4.scales_row_major(sf, rows, K, bn).view(torch.float8_e4m3fn), 1.0) * g.unsqueeze(-1)


def test_scale_tile_layout():
    from slopllm_b200.ops import fp4
    mats, rows, K = 3, 256, 512
    s = torch.randint(0, 127, (mats, rows, K // 16), dtype=torch.uint8, device=DEV)
    t = fp4.sf_tiles(s).cpu()
    s = s.cpu()
    kt_n = K // 64
    for mat, r, kb in [(0, 0, 0), (1, 37, 5), (2, 255, 31), (0, 128, 4), (2, 96, 7), (1, 200, 30)]:
        blk = mat * (rows // 128) + r // 128
        rr = r % 128
        off = (blk * kt_n + kb // 4) * 512 + (rr % 32) * 16 + (rr // 32) * 4 + kb % 4
        assert int(t[off]) == int(s[mat, r, kb]), (mat, r, kb)


@pytest.mark.parametrize("terms", [1, 3])
def test_quantize_rows_represents_the_input(terms):
    from slopllm_b200.ops import fp4
    M, K = 37, 1024
    x = (torch.randn(M, K, device=DEV) * torch.rand(M, 1, device=DEV) * 3).to(torch.bfloat16)
    x[5] = 0
    src = torch.randperm(M, device=DEV).to(torch.int32)
    q, sf, g = fp4.quantize_rows(x, src, terms=terms, bn=32)
    xs = x[src.long()].float()
    allrows = deq_rows(q, sf, g, 32)                    # rows m + j * M: the j-th term of row m
    rep = sum(allrows[j * M:(j + 1) * M] for j in range(terms))
    rel = ((rep - xs).norm(dim=1) / xs.norm(dim=1).clamp(min=1e-6))
    assert float(rel.max()) < (0.15 if terms == 1 else 2e-3), float(rel.max())
    assert float(rep[src.long() == 5].abs().max()) == 0.0
    # first term: the same scales and codes as the PyTorch definition of the format
    x0 = xs
    g_ref = x0.abs().amax(1) / (6 * 448)
    ok = g_ref > 0
    assert torch.allclose(g[:M][ok], g_ref[ok], rtol=1e-6)


@pytest.mark.parametrize("M,Nn,K,bn", [(8, 128, 256, 32), (100, 256, 1024, 128), (33, 384, 512, 64), (300, 128, 6144, 128), (64, 6144, 256, 64)])
def test_gemm_fp4_plain(M, Nn, K, bn):
    from slopllm_b200.ops import fp4, tcgen05
    g = torch.Generator(device=DEV).manual_seed(M + Nn)
    wq, ws, _ = quant.random_nvfp4((Nn, K), g, DEV)
    gA = torch.tensor([0.37], device=DEV)
    x = torch.randn(M, K, device=DEV, generator=g).to(torch.bfloat16)
    xq, sfb, gB = fp4.quantize_rows(x, bn=bn)
    y = fp4.gemm_fp4(wq, fp4.sf_tiles(ws), gA, xq, sfb, gB, fp4.OUT_F32, bn)
    torch.cuda.synchronize()
    tcgen05.check_errors(DEV)
    ref = deq_rows(xq, sfb, gB, bn) @ quant.nvfp4_dequantize(wq, ws, 0.37).t()
    close(y, ref, 2e-3, "fp4 gemm vs fp32 product of the quantised operands")
    # and the whole W4A4 path stays near the 16-bit activation product
    ref16 = x.float() @ quant.nvfp4_dequantize(wq, ws, 0.37).t()
    close(y, ref16, 0.12, "fp4 gemm vs 16-bit activations")


@pytest.mark.parametrize("pair", [False, True])
def test_gemm_fp4_grouped_ragged(pair):
    from slopllm_b200.ops import fp4, tcgen05
    G, Nn, K = 5, 256, 512
    counts = [70, 0, 129, 5, 33]
    M = sum(counts)
    g = torch.Generator(device=DEV).manual_seed(3)
    rows = 2 * Nn if pair else Nn
    wq, ws, _ = quant.random_nvfp4((G, rows, K), g, DEV)
    gA = (torch.rand(G, 2 if pair else 1, device=DEV, generator=g) + 0.5).squeeze(-1)
    x = torch.randn(M, K, device=DEV, generator=g).to(torch.bfloat16)
    off = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32, device=DEV)
    plan = fp4.group_plan(off, G, M, 64)
    xq, sfb, gB = fp4.quantize_rows(x, plan=plan)
    y = fp4.grouped_gemm_fp4(wq, fp4.sf_tiles(ws), gA, xq, sfb, gB, plan, Nn, pair, fp4.OUT_F32)
    torch.cuda.synchronize()
    tcgen05.check_errors(DEV)
    # the same rows quantised without groups give the same codes and scales (only the scale tiles move)
    xq2, sfb2, gB2 = fp4.quantize_rows(x, bn=64)
    assert torch.equal(xq, xq2) and torch.equal(gB, gB2)
    xd = deq_rows(xq2, sfb2, gB2, 64)
    ref = torch.empty(M, Nn, device=DEV)
    at = 0
    for e, n in enumerate(counts):
        wd = quant.nvfp4_dequantize(wq[e], ws[e], 1.0)
        h = xd[at:at + n] @ wd.t()
        if pair:
            gate, up = h[:, :Nn] * gA[e, 0], h[:, Nn:] * gA[e, 1]
            ref[at:at + n] = torch.nn.functional.silu(gate) * up
        else:
            ref[at:at + n] = h * gA[e]
        at += n
    close(y, ref, 3e-3, "grouped fp4 gemm")


def test_gather_of_quantised_rows_equals_quantising_the_gathered_rows():
    from slopllm_b200.ops import fp4
    T, K, G = 50, 512, 4
    g = torch.Generator(device=DEV).manual_seed(9)
    x = torch.randn(T, K, device=DEV, generator=g).to(torch.bfloat16)
    src = torch.randint(0, T, (173,), device=DEV, generator=g).to(torch.int32)
    off = torch.tensor([0, 60, 60, 100, 173], dtype=torch.int32, device=DEV)
    plan = fp4.group_plan(off, G, 173, 64)
    a = fp4.quantize_rows(x, src, plan=plan)
    b = fp4.gather_rows(*fp4.quantize_rows(x, bn=128), 128, src, plan)
    for u, v in zip(a, b):
        assert torch.equal(u, v)
