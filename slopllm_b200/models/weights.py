"""Weight containers, tensor-parallel sharding rules and random initialisation.

Parity: per-weight TP rules follow `src/glm51_model.ts:178-232` (lm_head column-split;
gate/up column-split; o_proj/down row-split; MLA q_b / k_nope / v_proj head-split;
everything else replicated) and the MLA re-layout at load time follows `:281-343`
(kv_b_proj split into the absorbed `k_nope` [h, Dn, R] and `v_proj` [h, R, Dv]).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from ..config import GlmMoeDsaConfig
from ..ops import quant


@dataclass
class LinearWeight:
    """`y = x @ W^T` weight: bf16/f32 dense, NVFP4 (packed u8 + e4m3 block scale + f32 global), or FP8 e4m3 with one
    fp32 scale per 128 x 128 block (`fp8_scale` [ceil(N/128), ceil(K/128)], the `weight_scale_inv` of FP8 checkpoints)."""

    weight: torch.Tensor
    scale: Optional[torch.Tensor] = None
    scale2: Optional[torch.Tensor] = None
    fp8_scale: Optional[torch.Tensor] = None

    @property
    def is_nvfp4(self) -> bool:
        return self.scale is not None

    @property
    def is_fp8(self) -> bool:
        return self.fp8_scale is not None

    @property
    def out_features(self) -> int:
        return self.weight.shape[0]

    @property
    def in_features(self) -> int:
        return self.weight.shape[1] * (2 if self.is_nvfp4 else 1)

    def dequant(self, dtype=torch.float32) -> torch.Tensor:
        if self.is_nvfp4:
            return quant.nvfp4_dequantize(self.weight, self.scale, self.scale2, dtype)
        if self.is_fp8:
            return quant.fp8_block_dequantize(self.weight, self.fp8_scale).to(dtype)
        return self.weight.to(dtype)

    def rows(self, lo: int, hi: int) -> "LinearWeight":
        """Column-parallel shard (split of the output features)."""
        if self.is_nvfp4:
            return LinearWeight(self.weight[lo:hi].contiguous(), self.scale[lo:hi].contiguous(), self.scale2)
        if self.is_fp8:
            assert lo % 128 == 0 and (hi % 128 == 0 or hi == self.weight.shape[0])
            return LinearWeight(self.weight[lo:hi].contiguous(), fp8_scale=self.fp8_scale[lo // 128:(hi + 127) // 128].contiguous())
        return LinearWeight(self.weight[lo:hi].contiguous())

    def cols(self, lo: int, hi: int) -> "LinearWeight":
        """Row-parallel shard (split of the input features; multiples of 16 for NVFP4)."""
        if self.is_nvfp4:
            assert lo % 16 == 0 and hi % 16 == 0
            return LinearWeight(self.weight[:, lo // 2:hi // 2].contiguous(),
                                self.scale[:, lo // 16:hi // 16].contiguous(), self.scale2)
        if self.is_fp8:
            assert lo % 128 == 0 and (hi % 128 == 0 or hi == self.weight.shape[1])
            return LinearWeight(self.weight[:, lo:hi].contiguous(), fp8_scale=self.fp8_scale[:, lo // 128:(hi + 127) // 128].contiguous())
        return LinearWeight(self.weight[:, lo:hi].contiguous())

    def to(self, device=None, dtype=None) -> "LinearWeight":
        w = self.weight.to(device=device)
        if not self.is_nvfp4 and not self.is_fp8 and dtype is not None:
            w = w.to(dtype)
        return LinearWeight(w, None if self.scale is None else self.scale.to(device),
                            None if self.scale2 is None else self.scale2.to(device),
                            None if self.fp8_scale is None else self.fp8_scale.to(device))

    @staticmethod
    def cat(parts: List["LinearWeight"]) -> "LinearWeight":
        """Concatenate along the output features (all dense, or all NVFP4 with equal global scale)."""
        if parts[0].is_nvfp4:
            return LinearWeight(torch.cat([p.weight for p in parts]), torch.cat([p.scale for p in parts]), parts[0].scale2)
        return LinearWeight(torch.cat([p.weight for p in parts]))

    def nbytes(self) -> int:
        n = self.weight.numel() * self.weight.element_size()
        if self.scale is not None:
            n += self.scale.numel()
        return n


@dataclass
class ExpertWeights:
    """Stacked SwiGLU experts.

    w13 `[E, 2*I, H]` (gate rows then up rows) and w2 `[E, H, I]`; NVFP4 (packed along the
    last dim, `s13`/`s2` e4m3 block scales, `g13 [E, 2]` / `g2 [E]` f32 global scales) or
    dense (scales None).  `I` is this rank's slice of the intermediate dim under TP, and `E`
    this rank's experts under EP (`expert_offset` = first global expert id held).
    """

    w13: torch.Tensor
    w2: torch.Tensor
    s13: Optional[torch.Tensor] = None
    s2: Optional[torch.Tensor] = None
    g13: Optional[torch.Tensor] = None
    g2: Optional[torch.Tensor] = None
    expert_offset: int = 0

    @property
    def is_nvfp4(self) -> bool:
        return self.s13 is not None

    @property
    def num_experts(self) -> int:
        return self.w13.shape[0]

    @property
    def hidden(self) -> int:
        return self.w2.shape[1]

    @property
    def inter(self) -> int:
        return self.w13.shape[1] // 2

    def dequant_expert(self, e: int):
        e = e - self.expert_offset
        if not self.is_nvfp4:
            return self.w13[e].to(torch.float32), self.w2[e].to(torch.float32)
        I = self.inter
        g = self.g13[e].to(torch.float32)
        w13 = quant.nvfp4_dequantize(self.w13[e], self.s13[e], 1.0)
        w13 = torch.cat([w13[:I] * g[0], w13[I:] * g[1]])
        return w13, quant.nvfp4_dequantize(self.w2[e], self.s2[e], self.g2[e])

    def tp_slice(self, rank: int, world: int) -> "ExpertWeights":
        """Slice the intermediate dim: gate/up column-parallel, down row-parallel."""
        I = self.inter
        Ir = I // world
        lo, hi = rank * Ir, (rank + 1) * Ir
        if self.is_nvfp4:
            assert Ir % 16 == 0
            w13 = torch.cat([self.w13[:, lo:hi], self.w13[:, I + lo:I + hi]], 1).contiguous()
            s13 = torch.cat([self.s13[:, lo:hi], self.s13[:, I + lo:I + hi]], 1).contiguous()
            return ExpertWeights(w13, self.w2[:, :, lo // 2:hi // 2].contiguous(), s13,
                                 self.s2[:, :, lo // 16:hi // 16].contiguous(), self.g13, self.g2, self.expert_offset)
        w13 = torch.cat([self.w13[:, lo:hi], self.w13[:, I + lo:I + hi]], 1).contiguous()
        return ExpertWeights(w13, self.w2[:, :, lo:hi].contiguous())

    def ep_slice(self, rank: int, world: int) -> "ExpertWeights":
        E = self.num_experts
        lo, hi = rank * (E // world), (rank + 1) * (E // world)
        pick = lambda t: None if t is None else t[lo:hi].contiguous()
        return ExpertWeights(pick(self.w13), pick(self.w2), pick(self.s13), pick(self.s2), pick(self.g13),
                             pick(self.g2), expert_offset=lo)

    def to(self, device=None, dtype=None) -> "ExpertWeights":
        mv = lambda t: None if t is None else t.to(device)
        w13, w2 = mv(self.w13), mv(self.w2)
        if not self.is_nvfp4 and dtype is not None:
            w13, w2 = w13.to(dtype), w2.to(dtype)
        return ExpertWeights(w13, w2, mv(self.s13), mv(self.s2), mv(self.g13), mv(self.g2), self.expert_offset)

    def nbytes(self) -> int:
        n = 0
        for t in (self.w13, self.w2, self.s13, self.s2):
            if t is not None:
                n += t.numel() * t.element_size()
        return n


@dataclass
class LayerWeights:
    """One decoder layer, already sharded for this rank and laid out for the fused kernels."""

    input_norm: torch.Tensor
    post_attn_norm: torch.Tensor
    w_qkv_a: LinearWeight            # rows: q_a | ckv | k_pe | (idx wk | idx weights_proj)
    q_a_norm: torch.Tensor
    kv_a_norm: torch.Tensor
    w_q_b: LinearWeight              # rows: local heads * (Dn + Dr) | (indexer wq_b)
    w_kn: torch.Tensor               # [h_local, Dn, R]
    w_v: torch.Tensor                # [h_local, R, Dv]
    o_proj: LinearWeight             # [H, h_local * Dv]
    idx_k_norm_w: Optional[torch.Tensor] = None
    idx_k_norm_b: Optional[torch.Tensor] = None
    has_indexer: bool = False
    # MLP
    mlp_w13: Optional[LinearWeight] = None     # dense: [2*I_local, H]
    mlp_w2: Optional[LinearWeight] = None      # dense: [H, I_local]
    router_w: Optional[torch.Tensor] = None    # [E, H]
    router_bias: Optional[torch.Tensor] = None # [E] f32
    experts: Optional[ExpertWeights] = None    # routed (TP-sliced or EP-sliced)
    shared: Optional[ExpertWeights] = None     # shared expert(s) as E=1 stack (TP-sliced)
    # MTP extras
    enorm: Optional[torch.Tensor] = None
    hnorm: Optional[torch.Tensor] = None
    eh_proj: Optional[LinearWeight] = None     # [H, 2H] (replicated)
    shared_head_norm: Optional[torch.Tensor] = None

    def nbytes(self) -> int:
        n = 0
        for v in self.__dict__.values():
            if isinstance(v, torch.Tensor):
                n += v.numel() * v.element_size()
            elif isinstance(v, (LinearWeight, ExpertWeights)):
                n += v.nbytes()
        return n


@dataclass
class ModelWeights:
    embed: torch.Tensor                       # [V, H] replicated
    layers: List[LayerWeights]                # num_hidden_layers (+ MTP layers at the end)
    final_norm: torch.Tensor
    lm_head: LinearWeight                     # [V / W, H] column shard
    vocab_offset: int = 0
    extra: Dict[str, torch.Tensor] = field(default_factory=dict)

    def nbytes(self) -> int:
        return (self.embed.numel() * self.embed.element_size() + self.lm_head.nbytes()
                + sum(l.nbytes() for l in self.layers))


# ---- random initialisation ------------------------------------------------------------------


def _gen(seed: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def _dense(shape, g, device, dtype, std=0.02) -> torch.Tensor:
    t = torch.empty(shape, device=device, dtype=torch.float32)
    t.normal_(0.0, std, generator=g)
    return t.to(dtype)


def _rand_linear(n, k, g, device, dtype, nvfp4: bool) -> LinearWeight:
    if nvfp4:
        return LinearWeight(*quant.random_nvfp4((n, k), g, device))
    return LinearWeight(_dense((n, k), g, device, dtype))


def _rand_experts(E, I, H, g, device, dtype, nvfp4: bool) -> ExpertWeights:
    if nvfp4:
        w13, s13, _ = quant.random_nvfp4((E, 2 * I, H), g, device)
        w2, s2, _ = quant.random_nvfp4((E, H, I), g, device)
        return ExpertWeights(w13, w2, s13, s2, torch.ones(E, 2, device=device), torch.ones(E, device=device))
    return ExpertWeights(_dense((E, 2 * I, H), g, device, dtype), _dense((E, H, I), g, device, dtype))


def random_layer(cfg: GlmMoeDsaConfig, layer: int, seed: int, device, dtype, tp_rank: int = 0, tp_world: int = 1,
                 ep: bool = False, exact: bool = True, is_mtp: bool = False) -> LayerWeights:
    """Random-init one layer.

    `exact=True` draws the *full* layer from (seed, layer) and slices it, so every TP degree
    sees the same model (tests compare TP=1 with TP=2).  `exact=False` draws only this
    rank's shard directly on `device` — the full-size benchmark model does not fit
    anywhere un-sharded.
    """
    W, r = tp_world, tp_rank
    H, R, Dn, Dr, Dv = cfg.hidden_size, cfg.kv_lora_rank, cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim
    h, hl = cfg.num_attention_heads, cfg.num_attention_heads // W
    Hi, Di = cfg.index_n_heads, cfg.index_head_dim
    full_idx = cfg.indexer_is_full(layer)
    if exact:
        g = _gen(seed * 1000003 + layer, "cpu")
        gdev = "cpu"
        hh, rr, WW = h, 0, 1
    else:
        g = _gen(seed * 1000003 + layer * 64 + r, device)
        gdev = device
        hh, rr, WW = hl, 0, 1      # generate local shapes directly
    # tensors that every rank holds in full (q_a / kv_a, indexer, router, MTP eh_proj) must be identical on all ranks:
    # they come from a generator that does not depend on the rank (slot 63 of the layer's seed range; ranks use 0..7)
    gr = g if exact else _gen(seed * 1000003 + layer * 64 + 63, device)
    ones = lambda n: torch.ones(n, device=gdev, dtype=dtype)

    parts = [_dense((cfg.q_lora_rank, H), gr, gdev, dtype), _dense((R, H), gr, gdev, dtype), _dense((Dr, H), gr, gdev, dtype)]
    wq_b = _dense((hh * (Dn + Dr), cfg.q_lora_rank), g, gdev, dtype)
    w_kn = _dense((hh, Dn, R), g, gdev, dtype)
    w_v = _dense((hh, R, Dv), g, gdev, dtype)
    o_proj = _rand_linear(H, hh * Dv, g, gdev, dtype, cfg.quant_o_proj)
    idx_parts = None
    if full_idx:
        idx_parts = [_dense((Di, H), gr, gdev, dtype), _dense((Hi, H), gr, gdev, dtype)]
        idx_wq_b = _dense((Hi * Di, cfg.q_lora_rank), gr, gdev, dtype)
    if exact and W > 1:
        wq_b = wq_b.reshape(h, Dn + Dr, -1)[r * hl:(r + 1) * hl].reshape(hl * (Dn + Dr), -1)
        w_kn, w_v = w_kn[r * hl:(r + 1) * hl], w_v[r * hl:(r + 1) * hl]
        o_proj = o_proj.cols(r * hl * Dv, (r + 1) * hl * Dv)
    if full_idx:
        parts += idx_parts
        wq_b = torch.cat([wq_b, idx_wq_b])
    lw = LayerWeights(
        input_norm=ones(H), post_attn_norm=ones(H), w_qkv_a=LinearWeight(torch.cat(parts)),
        q_a_norm=ones(cfg.q_lora_rank), kv_a_norm=ones(R), w_q_b=LinearWeight(wq_b.contiguous()),
        w_kn=w_kn.contiguous(), w_v=w_v.contiguous(), o_proj=o_proj, has_indexer=full_idx,
        idx_k_norm_w=ones(Di) if full_idx else None,
        idx_k_norm_b=torch.zeros(Di, device=gdev, dtype=dtype) if full_idx else None,
    )
    if cfg.is_moe_layer(layer):
        E, I = cfg.n_routed_experts, cfg.moe_intermediate_size
        lw.router_w = _dense((E, H), gr, gdev, dtype, std=0.1)
        lw.router_bias = torch.zeros(E, device=gdev, dtype=torch.float32)
        if exact:
            ex = _rand_experts(E, I, H, g, gdev, dtype, cfg.quant_experts)
            sh = _rand_experts(1, I * cfg.n_shared_experts, H, g, gdev, dtype, cfg.quant_experts) if cfg.n_shared_experts else None
            if W > 1:
                ex = ex.ep_slice(r, W) if ep else ex.tp_slice(r, W)
                sh = sh.tp_slice(r, W) if sh is not None else None
        else:
            if ep:
                ex = _rand_experts(E // W, I, H, g, gdev, dtype, cfg.quant_experts)
                ex.expert_offset = r * (E // W)
            else:
                ex = _rand_experts(E, I // W, H, g, gdev, dtype, cfg.quant_experts)
            sh = _rand_experts(1, I * cfg.n_shared_experts // W, H, g, gdev, dtype, cfg.quant_experts) if cfg.n_shared_experts else None
        lw.experts, lw.shared = ex, sh
    else:
        I = cfg.intermediate_size
        if exact:
            w13 = _rand_linear(2 * I, H, g, gdev, dtype, cfg.quant_dense_mlp)
            w2 = _rand_linear(H, I, g, gdev, dtype, cfg.quant_dense_mlp)
            if W > 1:
                Ir = I // W
                w13 = LinearWeight.cat([w13.rows(r * Ir, (r + 1) * Ir), w13.rows(I + r * Ir, I + (r + 1) * Ir)])
                w2 = w2.cols(r * Ir, (r + 1) * Ir)
        else:
            w13 = _rand_linear(2 * I // W, H, g, gdev, dtype, cfg.quant_dense_mlp)
            w2 = _rand_linear(H, I // W, g, gdev, dtype, cfg.quant_dense_mlp)
        lw.mlp_w13, lw.mlp_w2 = w13, w2
    if is_mtp:
        lw.enorm, lw.hnorm, lw.shared_head_norm = ones(H), ones(H), ones(H)
        lw.eh_proj = LinearWeight(_dense((H, 2 * H), gr, gdev, dtype))
    return layer_to(lw, device, dtype)


def layer_to(lw: LayerWeights, device, dtype) -> LayerWeights:
    out = {}
    for k, v in lw.__dict__.items():
        if isinstance(v, torch.Tensor):
            out[k] = v.to(device) if v.dtype in (torch.float32,) and k == "router_bias" else v.to(device=device, dtype=dtype)
        elif isinstance(v, (LinearWeight, ExpertWeights)):
            out[k] = v.to(device, dtype)
        else:
            out[k] = v
    return LayerWeights(**out)


def random_model(cfg: GlmMoeDsaConfig, seed: int = 0, device="cpu", dtype=torch.float32, tp_rank: int = 0,
                 tp_world: int = 1, ep: bool = False, exact: bool = True, with_mtp: bool = True) -> ModelWeights:
    """Random-init model (NVFP4 where the config says so), sharded for (tp_rank, tp_world)."""
    V, H = cfg.vocab_size, cfg.hidden_size
    g = _gen(seed * 1000003 + 999983, "cpu" if exact else device)
    gdev = "cpu" if exact else device
    embed = _dense((V, H), g, gdev, dtype, std=1.0)
    Vr = V // tp_world
    if exact:
        lm = _dense((V, H), g, gdev, dtype)[tp_rank * Vr:(tp_rank + 1) * Vr]
    else:
        lm = _dense((Vr, H), g, gdev, dtype)
    n_layers = cfg.num_hidden_layers + (cfg.num_nextn_predict_layers if with_mtp else 0)
    layers = [random_layer(cfg, i, seed, device, dtype, tp_rank, tp_world, ep, exact, is_mtp=i >= cfg.num_hidden_layers)
              for i in range(n_layers)]
    return ModelWeights(embed=embed.to(device=device, dtype=dtype), layers=layers,
                        final_norm=torch.ones(H, device=device, dtype=dtype),
                        lm_head=LinearWeight(lm.contiguous().to(device=device, dtype=dtype)), vocab_offset=tp_rank * Vr)
