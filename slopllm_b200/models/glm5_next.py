"""`glm5_next` (GLM-5.3-Flash class): config checks, weight workspace and the KDA attention
sub-layer with its per-sequence state; manifold hyper-connection helpers.

As in the reference, the decoder stack and its cache are not wired into the engine yet: the
checkpoint loads (text decoder only, MTP layers skipped) and the KDA / mHC building blocks run,
`forward_hidden` raises.  Reference: `src/glm53_flash_model.ts:1-174`, `src/kda.ts:1-71`,
`src/flash_hybrid_validation.ts:1-60`.
"""
from __future__ import annotations

import json
import os
import re
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from ..ops import recurrent as RC
from ..parallel.dist import ParallelContext

WEIGHT_PREFIX = "model.language_model."
LAYER_KINDS = ("linear_attention", "deepseek_sparse_attention", "indexed_attention")


@dataclass
class Glm5NextConfig:
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    vocab_size: int
    num_attention_heads: int
    num_key_value_heads: int
    q_lora_rank: int
    kv_lora_rank: int
    qk_nope_head_dim: int
    qk_rope_head_dim: int
    v_head_dim: int
    linear_num_heads: int
    linear_head_dim: int
    linear_conv_kernel_size: int
    linear_gate_lower_bound: float
    hc_mult: int
    hc_eps: float
    hc_sinkhorn_iters: int
    n_routed_experts: int
    n_shared_experts: int
    num_experts_per_tok: int
    moe_intermediate_size: int
    index_head_dim: int
    index_n_heads: int
    index_kpool: int
    layer_types: List[str] = field(default_factory=list)
    rms_norm_eps: float = 1e-5
    index_topk: int = 2048
    first_k_dense_replace: int = 0
    routed_scaling_factor: float = 1.0
    norm_topk_prob: bool = True
    n_group: int = 1
    topk_group: int = 1
    eos_token_ids: List[int] = field(default_factory=list)
    tie_word_embeddings: bool = False

    @classmethod
    def from_hf_dict(cls, raw: dict) -> "Glm5NextConfig":
        c = raw.get("text_config")
        if raw.get("model_type") != "glm5_next" or not c:
            raise ValueError("expected a glm5_next checkpoint with text_config")
        lin = c.get("linear_attn_config", {})
        eos = c.get("eos_token_id", [])
        cfg = cls(
            hidden_size=c.get("hidden_size"), intermediate_size=c.get("intermediate_size"), num_hidden_layers=c.get("num_hidden_layers"),
            vocab_size=c.get("vocab_size"), num_attention_heads=c.get("num_attention_heads"),
            num_key_value_heads=c.get("num_key_value_heads"), q_lora_rank=c.get("q_lora_rank"), kv_lora_rank=c.get("kv_lora_rank"),
            qk_nope_head_dim=c.get("qk_nope_head_dim"), qk_rope_head_dim=c.get("qk_rope_head_dim"), v_head_dim=c.get("v_head_dim"),
            linear_num_heads=c.get("linear_num_heads", lin.get("num_heads")), linear_head_dim=c.get("linear_head_dim", lin.get("head_dim")),
            linear_conv_kernel_size=c.get("linear_conv_kernel_dim", lin.get("short_conv_kernel_size")),
            linear_gate_lower_bound=c.get("linear_lower_bound", lin.get("gate_lower_bound")), hc_mult=c.get("hc_mult"),
            hc_eps=c.get("hc_eps"), hc_sinkhorn_iters=c.get("hc_sinkhorn_iters"), n_routed_experts=c.get("n_routed_experts"),
            n_shared_experts=c.get("n_shared_experts"), num_experts_per_tok=c.get("num_experts_per_tok"),
            moe_intermediate_size=c.get("moe_intermediate_size"), index_head_dim=c.get("index_head_dim"),
            index_n_heads=c.get("index_n_heads"), index_kpool=c.get("index_kpool"), layer_types=list(c.get("layer_types") or []),
            rms_norm_eps=c.get("rms_norm_eps", 1e-5), index_topk=c.get("index_topk", 2048),
            first_k_dense_replace=c.get("first_k_dense_replace", 0), routed_scaling_factor=c.get("routed_scaling_factor", 1.0),
            norm_topk_prob=c.get("norm_topk_prob", True), n_group=c.get("n_group", 1), topk_group=c.get("topk_group", 1),
            eos_token_ids=eos if isinstance(eos, list) else [eos], tie_word_embeddings=c.get("tie_word_embeddings", False))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for key in ("hidden_size", "intermediate_size", "num_hidden_layers", "vocab_size", "num_attention_heads",
                    "num_key_value_heads", "q_lora_rank", "kv_lora_rank", "linear_num_heads", "hc_sinkhorn_iters",
                    "n_routed_experts", "n_shared_experts", "num_experts_per_tok", "moe_intermediate_size", "index_head_dim",
                    "index_n_heads", "index_kpool"):
            v = getattr(self, key)
            if not isinstance(v, int) or isinstance(v, bool) or v < 1:
                raise ValueError(f"invalid glm5_next config {key}: {v!r}")
        if (self.hc_mult != 4 or self.qk_rope_head_dim != 0 or self.linear_head_dim != 128 or self.linear_conv_kernel_size != 4
                or self.linear_gate_lower_bound != -5):
            raise ValueError("unsupported glm5_next mHC / KDA / MLA geometry")
        if len(self.layer_types) != self.num_hidden_layers or any(t not in LAYER_KINDS for t in self.layer_types):
            raise ValueError("invalid glm5_next layer_types")


class KdaState:
    """Conv history of q, k, v and the recurrent state of one KDA layer, head-sharded under TP.
    The caller owns the mapping of sequences to state slots."""

    def __init__(self, batch_size: int, num_heads: int, device, world: int = 1):
        if batch_size < 1 or num_heads < 1 or num_heads % world:
            raise ValueError("KdaState requires a positive batch and heads divisible by the TP size")
        self.batch_size, self.num_heads = batch_size, num_heads // world
        width = self.num_heads * 128
        self.conv = torch.zeros(batch_size, 3 * width, 3, dtype=torch.float32, device=device)       # q | k | v channels, Kw - 1 = 3
        self.recurrent = torch.zeros(batch_size, self.num_heads, 128, 128, dtype=torch.float32, device=device)

    def reset(self) -> None:
        self.conv.zero_()
        self.recurrent.zero_()


@dataclass
class KdaWeights:
    q: torch.Tensor; k: torch.Tensor; v: torch.Tensor                       # [heads*128, H]
    q_conv: torch.Tensor; k_conv: torch.Tensor; v_conv: torch.Tensor        # [heads*128, 1, 4]
    f_a: torch.Tensor; f_b: torch.Tensor; beta: torch.Tensor                # low-rank forget gate, beta logits
    g_a: torch.Tensor; g_b: torch.Tensor; norm: torch.Tensor; out: torch.Tensor
    a_log: torch.Tensor; dt_bias: torch.Tensor                              # [heads] f32, [heads*128] f32


def kda_attention(hidden: torch.Tensor, w: KdaWeights, state: KdaState, qo_indptr: torch.Tensor, state_idx: torch.Tensor,
                  lower_bound: float = -5.0, eps: float = 1e-5) -> torch.Tensor:
    """Complete KDA sub-layer on normed hidden states [T, H]: projections, causal conv (kernel 4)
    with rolling state, low-rank forget gate, delta-rule scan with per-channel decay,
    sigmoid-gated RMSNorm, output projection.  `qo_indptr` partitions the tokens by sequence,
    `state_idx` names each sequence's state slot; decode and resumed prefill both work.
    The result is a partial sum under TP.  Reference `src/kda.ts:44-71`."""
    width, T = state.num_heads * 128, hidden.shape[0]
    for name in ("q", "k", "v", "f_b", "g_b"):
        if getattr(w, name).shape[0] != width:
            raise ValueError("kda_attention: projection width must match the state's heads")
    for name in ("q_conv", "k_conv", "v_conv"):
        if tuple(getattr(w, name).shape) != (width, 1, 4):
            raise ValueError("kda_attention: expected [heads * 128, 1, 4] convolution weights")
    dt = hidden.dtype
    lin = lambda x, m: (x.to(torch.float32) @ m.to(torch.float32).t()).to(dt)
    qkv = lin(hidden, torch.cat([w.q, w.k, w.v], 0))
    conv_w = torch.cat([w.q_conv, w.k_conv, w.v_conv], 0).reshape(3 * width, 4).to(dt)
    conv = RC.causal_conv1d(qkv.to(torch.bfloat16) if hidden.is_cuda else qkv, conv_w.to(torch.bfloat16) if hidden.is_cuda else conv_w,
                            None, state.conv, qo_indptr, state_idx, activation=True)
    forget = lin(lin(hidden, w.f_a), w.f_b).reshape(T, state.num_heads, 128)
    beta = lin(hidden, w.beta)
    core = RC.kda_scan(conv, forget.to(torch.bfloat16), beta.to(torch.bfloat16).contiguous(), w.a_log, w.dt_bias.reshape(state.num_heads, 128),
                       state.recurrent, qo_indptr, state_idx, state.num_heads, 128, 128, lower_bound)
    gate = lin(lin(hidden, w.g_a), w.g_b)
    gated = RC.rmsnorm_gated(core.reshape(T * state.num_heads, 128), gate.reshape(T * state.num_heads, 128).to(core.dtype),
                             w.norm.to(core.dtype), eps, sigmoid_gate=True)
    return lin(gated.reshape(T, width), w.out)


_COLUMN = re.compile(r"\.self_attn\.(q_proj|k_proj|v_proj|q_b_proj|kv_b_proj|b_proj|f_b_proj|g_b_proj|[qkv]_conv1d)$")
_COLUMN_VEC = re.compile(r"\.self_attn\.(A_log|dt_bias)$")
_COLUMN_MLP = re.compile(r"\.mlp\.(?:experts\.\d+\.|shared_experts\.)?(gate_proj|up_proj)$")
_ROW = re.compile(r"\.self_attn\.o_proj$|\.mlp\.(?:experts\.\d+\.|shared_experts\.)?down_proj$")


def weight_parallelism(name: str) -> str:
    """'column' | 'row' | 'replicated' for a checkpoint tensor (head-contiguous layouts are kept;
    MLA absorption belongs to the forward path).  Reference `src/glm53_flash_model.ts:108-121`."""
    if name == "lm_head.weight":
        return "column"
    if name == WEIGHT_PREFIX + "embed_tokens.weight":
        return "row"
    base = re.sub(r"\.(weight_scale|weight)$", "", name)
    if _COLUMN.search(base) or _COLUMN_VEC.search(base) or _COLUMN_MLP.search(base):
        return "column"
    if _ROW.search(base):
        return "row"
    return "replicated"


class Glm5NextModel:
    """Text-only weight workspace of a glm5_next checkpoint."""

    def __init__(self, cfg: Glm5NextConfig, ctx: Optional[ParallelContext] = None):
        self.cfg = cfg
        self.ctx = ctx or ParallelContext()
        if cfg.linear_num_heads % self.ctx.world or cfg.num_attention_heads % self.ctx.world:
            raise ValueError("glm5_next attention heads must be divisible by the TP size")
        self.tensors: Dict[str, torch.Tensor] = {}
        self.supports_prefix_sharing = False

    @classmethod
    def from_pretrained(cls, model_dir: str, ctx: Optional[ParallelContext] = None) -> "Glm5NextModel":
        from ..checkpoint.safetensors_io import SafetensorsFile
        from ..utils.model_path import list_safetensors_shards
        with open(os.path.join(model_dir, "config.json")) as f:
            model = cls(Glm5NextConfig.from_hf_dict(json.load(f)), ctx)
        for path in list_safetensors_shards(model_dir):
            sf = SafetensorsFile(path)
            for name in sf.names():
                model.load_tensor(name, sf.tensor(name), sf.meta(name).dtype)
            sf.close()
        return model

    def load_tensor(self, name: str, t: torch.Tensor, dtype_name: str = "BF16") -> None:
        if name.startswith("model.visual."):
            return
        m = re.match(r"^model\.language_model\.layers\.(\d+)\.", name)
        if m and int(m.group(1)) >= self.cfg.num_hidden_layers:
            return                                      # MTP layers (incl. their MXFP8 experts) are not loaded
        if name != "lm_head.weight" and not name.startswith(WEIGHT_PREFIX):
            raise ValueError(f"unsupported glm5_next tensor: {name}")
        if ".nvfp4_csf_" in name or (dtype_name == "F8_E4M3" and not name.endswith(".weight_scale")):
            raise ValueError(f"the glm5_next loader expects BF16 linears and uncompressed NVFP4 experts: {name}")
        par, W, r = weight_parallelism(name), self.ctx.world, self.ctx.rank
        if W > 1 and par == "column":
            n = t.shape[0] // W
            t = t[r * n:(r + 1) * n]
        elif W > 1 and par == "row" and t.dim() >= 2:
            n = t.shape[1] // W
            t = t[:, r * n:(r + 1) * n]
        self.tensors[name] = t.contiguous().to(self.ctx.device)

    def kda_weights(self, layer: int) -> KdaWeights:
        if self.cfg.layer_types[layer] != "linear_attention":
            raise ValueError(f"layer {layer} is not KDA")
        p = f"{WEIGHT_PREFIX}layers.{layer}.self_attn."

        def get(suffix):
            if p + suffix not in self.tensors:
                raise KeyError(f"missing KDA weight: {p}{suffix}")
            return self.tensors[p + suffix]

        return KdaWeights(q=get("q_proj.weight"), k=get("k_proj.weight"), v=get("v_proj.weight"), q_conv=get("q_conv1d.weight"),
                          k_conv=get("k_conv1d.weight"), v_conv=get("v_conv1d.weight"), f_a=get("f_a_proj.weight"),
                          f_b=get("f_b_proj.weight"), beta=get("b_proj.weight"), g_a=get("g_a_proj.weight"), g_b=get("g_b_proj.weight"),
                          norm=get("o_norm.weight"), out=get("o_proj.weight"), a_log=get("A_log").to(torch.float32),
                          dt_bias=get("dt_bias").to(torch.float32))

    def allocate_cache(self, num_pages: int):
        raise NotImplementedError("the glm5_next hybrid chat cache is not implemented")

    def forward_hidden(self, st, cache):
        raise NotImplementedError("the glm5_next forward pass is not implemented")


__all__ = ["Glm5NextConfig", "Glm5NextModel", "KdaState", "KdaWeights", "kda_attention", "weight_parallelism", "R"]
