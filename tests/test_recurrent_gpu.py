"""sm_100a kernels of the dense / hybrid families against their fp32 definitions: the same op
wrapper is run on CUDA tensors (native kernel) and on CPU copies (plain PyTorch)."""
import pytest
import torch

from slopllm_b200.ops import dense as D
from slopllm_b200.ops import recurrent as RC

pytestmark = pytest.mark.gpu


def rel_err(a, b):
    a, b = a.to(torch.float32).cpu(), b.to(torch.float32).cpu()
    return ((a - b).abs().max() / b.abs().max().clamp(min=1e-6)).item()


def gen(seed):
    return torch.Generator().manual_seed(seed)


@pytest.mark.parametrize("dk,dv,h", [(128, 128, 4), (64, 64, 2)])
@pytest.mark.parametrize("lens", [[1, 1, 1], [37, 5, 64]])
def test_gdn_scan(dk, dv, h, lens):
    g = gen(1)
    T, B = sum(lens), len(lens)
    qkv = torch.randn(T, h * (2 * dk + dv), generator=g).to(torch.bfloat16)
    a = torch.randn(T, h, generator=g).to(torch.bfloat16)
    b = torch.randn(T, h, generator=g).to(torch.bfloat16)
    A_log, dt_bias = torch.randn(h, generator=g) * 0.5, torch.randn(h, generator=g) * 0.1
    state = torch.randn(B + 2, h, dk, dv, generator=g) * 0.1
    ind = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    sidx = torch.tensor([2, 0, 3][:B], dtype=torch.int32)
    s_cpu, s_gpu = state.clone(), state.clone().cuda()
    want = RC.gdn_scan(qkv, a, b, A_log, dt_bias, s_cpu, ind, sidx, h, dk, dv)
    got = RC.gdn_scan(qkv.cuda(), a.cuda(), b.cuda(), A_log.cuda(), dt_bias.cuda(), s_gpu, ind.cuda(), sidx.cuda(), h, dk, dv)
    assert rel_err(got, want) < 2e-2
    assert rel_err(s_gpu, s_cpu) < 1e-3


def test_kda_scan():
    g = gen(2)
    h, dk, dv, lens = 2, 128, 128, [9, 20]
    T = sum(lens)
    qkv = (torch.randn(T, h * (2 * dk + dv), generator=g) * 0.3).to(torch.bfloat16)
    forget = torch.randn(T, h, dk, generator=g).to(torch.bfloat16)
    b = torch.randn(T, h, generator=g).to(torch.bfloat16)
    A_log, dt_bias = torch.randn(h, generator=g) * 0.3, torch.randn(h, dk, generator=g) * 0.2
    state = torch.zeros(2, h, dk, dv)
    ind = torch.tensor([0, 9, 29], dtype=torch.int32)
    sidx = torch.tensor([1, 0], dtype=torch.int32)
    s_cpu, s_gpu = state.clone(), state.clone().cuda()
    want = RC.kda_scan(qkv, forget, b, A_log, dt_bias, s_cpu, ind, sidx, h, dk, dv, -5.0)
    got = RC.kda_scan(qkv.cuda(), forget.cuda(), b.cuda(), A_log.cuda(), dt_bias.cuda(), s_gpu, ind.cuda(), sidx.cuda(), h, dk, dv, -5.0)
    assert rel_err(got, want) < 2e-2
    assert rel_err(s_gpu, s_cpu) < 2e-3


def test_causal_conv1d_prefill_then_update():
    g = gen(3)
    C_, Kw = 320, 4
    w = (torch.randn(C_, Kw, generator=g) * 0.5).to(torch.bfloat16)
    x1 = torch.randn(45, C_, generator=g).to(torch.bfloat16)
    x2 = torch.randn(2, C_, generator=g).to(torch.bfloat16)
    st_c, st_g = torch.zeros(3, C_, Kw - 1), torch.zeros(3, C_, Kw - 1).cuda()
    ind1, sid = torch.tensor([0, 30, 45], dtype=torch.int32), torch.tensor([2, 1], dtype=torch.int32)
    ind2 = torch.tensor([0, 1, 2], dtype=torch.int32)
    for x, ind in ((x1, ind1), (x2, ind2)):
        want = RC.causal_conv1d(x, w, None, st_c, ind, sid)
        got = RC.causal_conv1d(x.cuda(), w.cuda(), None, st_g, ind.cuda(), sid.cuda())
        assert rel_err(got, want) < 1e-2
    assert rel_err(st_g, st_c) < 1e-6


@pytest.mark.parametrize("sig", [False, True])
def test_rmsnorm_gated(sig):
    g = gen(4)
    x = torch.randn(50, 128, generator=g).to(torch.bfloat16)
    gate = torch.randn(50, 128, generator=g).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(128, generator=g)).to(torch.bfloat16)
    assert rel_err(RC.rmsnorm_gated(x.cuda(), gate.cuda(), w.cuda(), 1e-6, sig), RC.rmsnorm_gated(x, gate, w, 1e-6, sig)) < 1e-2


def test_mhc():
    g = gen(5)
    T, H = 6, 512
    x = torch.randn(T, 4, H, generator=g).to(torch.bfloat16)
    fn = (torch.randn(24, 4 * H, generator=g) * 0.05).to(torch.bfloat16)
    base, scale = torch.randn(24, generator=g) * 0.5, torch.tensor([0.7, 1.3, 0.9])
    c_c, p_c, m_c = RC.mhc_pre(x, fn, base, scale, 1e-6, 1e-6, 20)
    c_g, p_g, m_g = RC.mhc_pre(x.cuda(), fn.cuda(), base.cuda(), scale.cuda(), 1e-6, 1e-6, 20)
    assert rel_err(c_g, c_c) < 1e-2 and rel_err(p_g, p_c) < 1e-3 and rel_err(m_g, m_c) < 1e-3
    # the mixing matrix is (close to) doubly stochastic
    assert (m_c.sum(-2) - 1).abs().max() < 1e-3
    y = torch.randn(T, H, generator=g).to(torch.bfloat16)
    assert rel_err(RC.mhc_post(x.cuda(), y.cuda(), p_c.cuda(), m_c.cuda()), RC.mhc_post(x, y, p_c, m_c)) < 1e-2
    assert rel_err(RC.mhc_streams(x.cuda(), False), RC.mhc_streams(x, False)) < 1e-2
    assert torch.equal(RC.mhc_streams(y.cuda(), True).cpu(), RC.mhc_streams(y, True))


def _paged_setup(g, B, lens, n_kv, hd, page=64):
    pages_per = [(-(-l // page)) for l in lens]
    total = sum(pages_per) + 1
    perm = torch.randperm(total - 1, generator=g) + 1
    pt = torch.zeros(B, max(pages_per), dtype=torch.int32)
    o = 0
    for b, n in enumerate(pages_per):
        pt[b, :n] = perm[o:o + n].to(torch.int32)
        o += n
    k_cache = torch.randn(total * page, n_kv, hd, generator=g).to(torch.bfloat16)
    v_cache = torch.randn(total * page, n_kv, hd, generator=g).to(torch.bfloat16)
    return pt, k_cache, v_cache


@pytest.mark.parametrize("hd,heads,n_kv", [(128, 8, 2), (64, 4, 4), (128, 16, 1)])
def test_paged_attention_decode_and_prefill(hd, heads, n_kv):
    g = gen(6)
    lens = [300, 77, 1025]
    B = len(lens)
    pt, kc, vc = _paged_setup(g, B, lens, n_kv, hd)
    scale = hd ** -0.5
    # decode: one query per sequence at its last position
    q = torch.randn(B, heads, hd, generator=g).to(torch.bfloat16)
    pos = torch.tensor([l - 1 for l in lens], dtype=torch.int32)
    bi = torch.arange(B, dtype=torch.int32)
    want = D.paged_attention(q, kc, vc, pos, bi, pt, 64, scale)
    got = D.paged_attention(q.cuda(), kc.cuda(), vc.cuda(), pos.cuda(), bi.cuda(), pt.cuda(), 64, scale, max_kv_len=max(lens))
    assert rel_err(got, want) < 2e-2
    # prefill: the last 70 / 77 / 130 positions of each sequence as one batch of query ranges
    qlens = [70, 77, 130]
    T = sum(qlens)
    q = torch.randn(T, heads, hd, generator=g).to(torch.bfloat16)
    pos = torch.cat([torch.arange(l - n, l) for l, n in zip(lens, qlens)]).to(torch.int32)
    bi = torch.cat([torch.full((n,), b) for b, n in enumerate(qlens)]).to(torch.int32)
    ind = torch.tensor([0, 70, 147, 277], dtype=torch.int32)
    want = D.paged_attention(q, kc, vc, pos, bi, pt, 64, scale)
    got = D.paged_attention(q.cuda(), kc.cuda(), vc.cuda(), pos.cuda(), bi.cuda(), pt.cuda(), 64, scale, qo_indptr=ind.cuda(),
                            max_q=max(qlens))
    assert rel_err(got, want) < 2e-2


def test_qk_norm_rope_cache_write():
    g = gen(7)
    T, heads, n_kv, hd, rope = 9, 4, 2, 128, 64
    q = torch.randn(T, heads * hd * 2, generator=g).to(torch.bfloat16)        # gate packed after each head's q
    k = torch.randn(T, n_kv * hd, generator=g).to(torch.bfloat16)
    v = torch.randn(T, n_kv * hd, generator=g).to(torch.bfloat16)
    qn = (1 + 0.1 * torch.randn(hd, generator=g)).to(torch.bfloat16)
    kn = (1 + 0.1 * torch.randn(hd, generator=g)).to(torch.bfloat16)
    pos = torch.arange(60, 60 + T, dtype=torch.int32)
    bi = torch.zeros(T, dtype=torch.int32)
    pt = torch.tensor([[3, 1]], dtype=torch.int32)
    kc_c, vc_c = torch.zeros(4 * 64, n_kv, hd, dtype=torch.bfloat16), torch.zeros(4 * 64, n_kv, hd, dtype=torch.bfloat16)
    kc_g, vc_g = kc_c.clone().cuda(), vc_c.clone().cuda()
    want = D.qk_norm_rope_cache(q, k, v, qn, kn, pos, bi, pt, 64, kc_c, vc_c, heads, n_kv, hd, rope, 1e6, 1e-6, q_stride=2 * hd)
    got = D.qk_norm_rope_cache(q.cuda(), k.cuda(), v.cuda(), qn.cuda(), kn.cuda(), pos.cuda(), bi.cuda(), pt.cuda(), 64, kc_g, vc_g,
                               heads, n_kv, hd, rope, 1e6, 1e-6, q_stride=2 * hd)
    assert rel_err(got, want) < 1e-2
    assert rel_err(kc_g, kc_c) < 1e-2 and rel_err(vc_g, vc_c) < 1e-6


def test_quantize_fp8_and_prefetch():
    from slopllm_b200.ops import misc
    g = gen(8)
    x = (torch.randn(37, 300, generator=g) * 3).to(torch.bfloat16)
    q_c, s_c = misc.quantize_fp8(x)
    q_g, s_g = misc.quantize_fp8(x.cuda())
    assert torch.equal(s_g.cpu(), s_c)
    deq = lambda q, s: q.view(torch.float8_e4m3fn).to(torch.float32) * s.repeat_interleave(128, 1)[:, :300]
    assert rel_err(deq(q_g.cpu(), s_g.cpu()), deq(q_c, s_c)) < 1e-6
    assert rel_err(deq(q_c, s_c), x) < 0.07
    misc.prefetch_l2(x.cuda())                       # must simply run
    torch.cuda.synchronize()


def test_gather_topk_ckv():
    from slopllm_b200.ops import misc, quant
    g = gen(9)
    R, Dr, group, n, T, k = 512, 64, 128, 300, 5, 64
    cache = quant.pack_kv_rows(torch.randn(n, R, generator=g), torch.randn(n, Dr, generator=g), group)
    slots = torch.randint(0, n, (T, k), generator=g).to(torch.int32)
    lengths = torch.tensor([64, 10, 0, 33, 64], dtype=torch.int32)
    d_c, w_c, u_c = misc.gather_topk_ckv(cache, slots, lengths, R, Dr, group)
    d_g, w_g, u_g = misc.gather_topk_ckv(cache.cuda(), slots.cuda(), lengths.cuda(), R, Dr, group)
    assert u_c == u_g and torch.equal(w_g.cpu(), w_c)
    assert rel_err(d_g, d_c) < 1e-2
    # fan-out consistency: row where[t, j] of the dense buffer is the row of slot slots[t, j]
    ckv, kpe = quant.unpack_kv_rows(cache[slots[0, 3].long()].unsqueeze(0), R, Dr, group)
    assert rel_err(d_g[w_g[0, 3].long()].cpu(), torch.cat([ckv, kpe], 1)[0]) < 1e-2
