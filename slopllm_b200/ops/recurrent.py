"""Recurrent sub-layer ops of the hybrid families: Gated DeltaNet (Qwen3.5), KDA and manifold
hyper-connections (glm5_next).  CUDA tensors run the sm_100a kernels of `csrc/recurrent.cu`;
CPU tensors run the fp32 definitions in `ops/reference.py` (the oracle of the GPU tests).
"""
from __future__ import annotations

import ctypes as C

import torch

from . import reference as R


class GdnParams(C.Structure):
    _fields_ = [("out", C.c_void_p), ("state", C.c_void_p), ("qkv", C.c_void_p), ("ld_qkv", C.c_int), ("a", C.c_void_p),
                ("b", C.c_void_p), ("A_log", C.c_void_p), ("dt_bias", C.c_void_p), ("g", C.c_void_p), ("qo_indptr", C.c_void_p),
                ("state_idx", C.c_void_p), ("h", C.c_int), ("dk", C.c_int), ("dv", C.c_int), ("normalize_qk", C.c_int),
                ("lower_bound", C.c_float), ("norm_eps", C.c_float)]


def _native():
    from . import native as N
    return N


def _split_qkv(qkv, h, dk, dv):
    T = qkv.shape[0]
    q = qkv[:, :h * dk].reshape(T, h, dk)
    k = qkv[:, h * dk:2 * h * dk].reshape(T, h, dk)
    v = qkv[:, 2 * h * dk:2 * h * dk + h * dv].reshape(T, h, dv)
    return q, k, v


def gdn_scan(qkv, a, b, A_log, dt_bias, state, qo_indptr, state_idx, h: int, dk: int, dv: int):
    """Gated DeltaNet over the token ranges of B sequences (a decode step is one token each).

    qkv [T, h*dk | h*dk | h*dv] (conv output), a/b [T, h], A_log/dt_bias [h] fp32, state
    [slots, h, dk, dv] fp32 updated in place, qo_indptr [B+1], state_idx [B].  q is
    L2-normalised and scaled by dk^-0.5, k L2-normalised, beta = sigmoid(b),
    decay = exp(-exp(A_log) * softplus(a + dt_bias)).  Returns [T, h, dv] bf16.
    """
    T = qkv.shape[0]
    if qkv.is_cuda:
        N = _native()
        out = torch.empty(T, h, dv, dtype=torch.bfloat16, device=qkv.device)
        p = GdnParams(out=out.data_ptr(), state=state.data_ptr(), qkv=qkv.data_ptr(), ld_qkv=qkv.stride(0), a=a.data_ptr(),
                      b=b.data_ptr(), A_log=A_log.data_ptr(), dt_bias=dt_bias.data_ptr(), g=0, qo_indptr=qo_indptr.data_ptr(),
                      state_idx=state_idx.data_ptr(), h=h, dk=dk, dv=dv, normalize_qk=1, lower_bound=0.0, norm_eps=1e-8)
        N.call("sl_delta_scan", C.byref(p), qo_indptr.numel() - 1, N.stream())
        return out
    q, k, v = _split_qkv(qkv.to(torch.float32), h, dk, dv)
    q = q * torch.rsqrt((q * q).sum(-1, keepdim=True) + 1e-8) * dk ** -0.5
    k = k * torch.rsqrt((k * k).sum(-1, keepdim=True) + 1e-8)
    beta = torch.sigmoid(b.to(torch.float32))
    g = -torch.exp(A_log.to(torch.float32)) * torch.nn.functional.softplus(a.to(torch.float32) + dt_bias.to(torch.float32))
    out = torch.empty(T, h, dv, dtype=torch.float32, device=qkv.device)
    ind = qo_indptr.tolist()
    for bi in range(len(ind) - 1):
        lo, hi = ind[bi], ind[bi + 1]
        if hi > lo:
            slot = int(state_idx[bi])
            out[lo:hi], state[slot] = R.gdn_recurrent(q[lo:hi], k[lo:hi], v[lo:hi], g[lo:hi], beta[lo:hi], state[slot])
    return out.to(torch.bfloat16)


def kda_scan(qkv, forget, b, A_log, dt_bias, state, qo_indptr, state_idx, h: int, dk: int, dv: int, lower_bound: float):
    """KDA recurrence: as :func:`gdn_scan` but with a per-channel decay
    exp(lower_bound * sigmoid(exp(A_log[h]) * (forget[t, h, :] + dt_bias[h, :]))), lower_bound < 0.
    qkv [T, h*dk | h*dk | h*dv] (conv outputs), forget [T, h, dk] bf16, b [T, h], dt_bias [h, dk] fp32."""
    if not lower_bound < 0:
        raise ValueError("kda_scan: the gate lower bound must be negative and finite")
    T = qkv.shape[0]
    if qkv.is_cuda:
        N = _native()
        out = torch.empty(T, h, dv, dtype=torch.bfloat16, device=qkv.device)
        forget = forget.to(torch.bfloat16).contiguous()
        p = GdnParams(out=out.data_ptr(), state=state.data_ptr(), qkv=qkv.data_ptr(), ld_qkv=qkv.stride(0), a=0, b=b.data_ptr(),
                      A_log=A_log.data_ptr(), dt_bias=dt_bias.contiguous().data_ptr(), g=forget.data_ptr(),
                      qo_indptr=qo_indptr.data_ptr(), state_idx=state_idx.data_ptr(), h=h, dk=dk, dv=dv, normalize_qk=1,
                      lower_bound=float(lower_bound), norm_eps=1e-6)
        N.call("sl_delta_scan", C.byref(p), qo_indptr.numel() - 1, N.stream())
        return out
    q, k, v = _split_qkv(qkv.to(torch.float32), h, dk, dv)
    out = torch.empty(T, h, dv, dtype=torch.float32, device=qkv.device)
    ind = qo_indptr.tolist()
    for bi in range(len(ind) - 1):
        lo, hi = ind[bi], ind[bi + 1]
        if hi > lo:
            slot = int(state_idx[bi])
            out[lo:hi], state[slot] = R.kda_scan(q[lo:hi], k[lo:hi], v[lo:hi], forget[lo:hi].reshape(hi - lo, h, dk), b[lo:hi], A_log,
                                                 dt_bias.reshape(h, dk), state[slot], lower_bound)
    return out.to(torch.bfloat16)


def causal_conv1d(x, weight, bias, state, qo_indptr, state_idx, activation: bool = True):
    """Depthwise causal conv over each sequence's tokens with rolling state [slots, C, Kw-1]
    (fp32, updated in place).  x [T, C] -> [T, C] bf16."""
    T, Cc = x.shape
    Kw = weight.shape[1]
    if x.is_cuda:
        N = _native()
        y = torch.empty(T, Cc, dtype=torch.bfloat16, device=x.device)
        N.call("sl_causal_conv1d", y.data_ptr(), state.data_ptr(), x.data_ptr(), weight.data_ptr(), N.ptr(bias),
               qo_indptr.data_ptr(), state_idx.data_ptr(), qo_indptr.numel() - 1, Cc, Kw, x.stride(0), int(activation), N.stream())
        return y
    y = torch.empty(T, Cc, dtype=torch.float32, device=x.device)
    ind = qo_indptr.tolist()
    for bi in range(len(ind) - 1):
        lo, hi = ind[bi], ind[bi + 1]
        if hi > lo:
            slot = int(state_idx[bi])
            y[lo:hi], state[slot] = R.causal_conv1d(x[lo:hi], weight, bias, state[slot], activation)
    return y.to(torch.bfloat16)


def rmsnorm_gated(x, gate, weight, eps: float, sigmoid_gate: bool = False):
    """rmsnorm(x) * w * silu(gate)  (sigmoid(gate) for KDA) over the last dim; x, gate [rows, D]."""
    if x.is_cuda:
        N = _native()
        x, gate = x.contiguous(), gate.contiguous()
        out = torch.empty_like(x)
        N.call("sl_rmsnorm_gated", out.data_ptr(), x.data_ptr(), gate.data_ptr(), weight.data_ptr(), x.shape[0], x.shape[1],
               float(eps), int(sigmoid_gate), N.stream())
        return out
    f = R.kda_norm if sigmoid_gate else R.rmsnorm_gated
    return f(x, gate, weight, eps).to(x.dtype)


def mhc_pre(x, fn, base, scale, norm_eps: float, hc_eps: float, iters: int):
    """x [T, 4, H] bf16 residual streams -> (collapsed [T, H] bf16, post [T, 4] f32, comb [T, 4, 4] f32)."""
    if x.dim() != 3 or x.shape[1] != 4 or not norm_eps > 0 or not hc_eps > 0 or iters < 1:
        raise ValueError("mhc_pre: expected [tokens, 4, hidden] and positive epsilons / iteration count")
    T, _, H = x.shape
    if tuple(fn.shape) != (24, 4 * H) or base.numel() != 24 or scale.numel() != 3:
        raise ValueError("mhc_pre: expected fn [24, 4*hidden], base [24], scale [3]")
    if x.is_cuda:
        N = _native()
        collapsed = torch.empty(T, H, dtype=torch.bfloat16, device=x.device)
        post = torch.empty(T, 4, dtype=torch.float32, device=x.device)
        comb = torch.empty(T, 4, 4, dtype=torch.float32, device=x.device)
        N.call("sl_mhc_pre", collapsed.data_ptr(), post.data_ptr(), comb.data_ptr(), x.to(torch.bfloat16).contiguous().data_ptr(),
               fn.to(torch.bfloat16).contiguous().data_ptr(), base.to(torch.float32).contiguous().data_ptr(),
               scale.to(torch.float32).contiguous().data_ptr(), T, H, float(norm_eps), float(hc_eps), int(iters), N.stream())
        return collapsed, post, comb
    collapsed, post, comb = R.mhc_pre(x, fn, base, scale, norm_eps, hc_eps, iters)
    return collapsed.to(torch.bfloat16), post, comb


def mhc_post(residual, block, post, comb):
    """residual [T, 4, H], block [T, H] -> new streams [T, 4, H] bf16."""
    if residual.dim() != 3 or residual.shape[1] != 4:
        raise ValueError("mhc_post: expected [tokens, 4, hidden]")
    if residual.is_cuda:
        N = _native()
        T, _, H = residual.shape
        out = torch.empty(T, 4, H, dtype=torch.bfloat16, device=residual.device)
        N.call("sl_mhc_post", out.data_ptr(), residual.to(torch.bfloat16).contiguous().data_ptr(),
               block.to(torch.bfloat16).contiguous().data_ptr(), post.contiguous().data_ptr(), comb.contiguous().data_ptr(), T, H,
               N.stream())
        return out
    return R.mhc_post(residual, block, post, comb).to(torch.bfloat16)


def mhc_streams(x, expand: bool):
    """expand: [T, H] -> [T, 4, H] (copies); collapse: [T, 4, H] -> [T, H] (mean)."""
    if (x.dim() != 2) if expand else (x.dim() != 3 or x.shape[1] != 4):
        raise ValueError("mhc_streams: expected [tokens, hidden] to expand or [tokens, 4, hidden] to collapse")
    if x.is_cuda:
        N = _native()
        T, H = x.shape[0], x.shape[-1]
        out = torch.empty((T, 4, H) if expand else (T, H), dtype=torch.bfloat16, device=x.device)
        N.call("sl_mhc_streams", out.data_ptr(), x.to(torch.bfloat16).contiguous().data_ptr(), T, H, int(expand), N.stream())
        return out
    return R.mhc_streams(x, expand).to(torch.bfloat16)
