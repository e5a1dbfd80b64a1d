"""Dense and hybrid model families served next to glm_moe_dsa: Qwen3 (grouped-query attention,
per-head q/k RMSNorm, optional FP8 block-quantised linears) and Qwen3.5 (Gated DeltaNet
linear-attention layers interleaved with gated full-attention layers).

One `DenseModel` class covers both: a layer is either "full_attention" or "linear_attention".
It plugs into the same `Engine` / scheduler as the flagship model (same `forward_hidden`,
`compute_logits`, `allocate_cache` surface) and shards like it under tensor parallelism
(q/k/v/gate/up and the GDN input projections by columns, o/down/out by rows).

Reference: `src/qwen3_model.ts:1-187`, `src/qwen35_model.ts:1-467`.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from ..config import PAGE_SIZE
from ..ops import dense as D
from ..ops import get_ops, recurrent as RC
from ..parallel.dist import Comm, ParallelContext
from ..utils.tracing import traced
from .weights import LinearWeight


@dataclass
class DenseConfig:
    model_type: str = "qwen3"
    hidden_size: int = 1024
    intermediate_size: int = 3072
    num_hidden_layers: int = 28
    num_attention_heads: int = 16
    num_key_value_heads: int = 8
    head_dim: int = 128
    vocab_size: int = 151936
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    eos_token_ids: List[int] = field(default_factory=lambda: [151645])
    # Qwen3.5
    partial_rotary_factor: float = 1.0
    attn_output_gate: bool = False
    layer_types: List[str] = field(default_factory=list)
    linear_num_key_heads: int = 16
    linear_key_head_dim: int = 128
    linear_num_value_heads: int = 16
    linear_value_head_dim: int = 128
    linear_conv_kernel_dim: int = 4
    gemma_norm: bool = False           # norm weights are stored as (w - 1)
    weight_prefix: str = "model."
    num_nextn_predict_layers: int = 0

    def __post_init__(self):
        if not self.layer_types:
            self.layer_types = ["full_attention"] * self.num_hidden_layers
        if len(self.layer_types) != self.num_hidden_layers:
            raise ValueError("layer_types must name every layer")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ValueError("num_attention_heads must be a multiple of num_key_value_heads")
        if "linear_attention" in self.layer_types and self.linear_num_value_heads != self.linear_num_key_heads:
            raise ValueError("Gated DeltaNet layers need linear_num_value_heads == linear_num_key_heads")

    @property
    def rope_dim(self) -> int:
        return int(self.head_dim * self.partial_rotary_factor) // 2 * 2

    @property
    def scaling(self) -> float:
        return self.head_dim ** -0.5

    @property
    def conv_dim(self) -> int:
        return self.linear_num_key_heads * (2 * self.linear_key_head_dim + self.linear_value_head_dim)

    @classmethod
    def from_hf_dict(cls, raw: dict) -> "DenseConfig":
        """Qwen3 reads the top level; Qwen3.5 nests the decoder under `text_config` and the
        rotary settings under `rope_parameters` (`src/qwen35_model.ts:73-113`)."""
        mt = raw.get("model_type", "qwen3")
        if mt in ("qwen3_5", "qwen3_5_text"):
            tc = raw.get("text_config", raw)
            rp = tc.get("rope_parameters", {})
            eos = raw.get("eos_token_id", tc.get("eos_token_id", 248044))
            return cls(model_type="qwen3_5", hidden_size=tc["hidden_size"], intermediate_size=tc["intermediate_size"],
                       num_hidden_layers=tc["num_hidden_layers"], num_attention_heads=tc["num_attention_heads"],
                       num_key_value_heads=tc["num_key_value_heads"], head_dim=tc["head_dim"], vocab_size=tc["vocab_size"],
                       rms_norm_eps=tc.get("rms_norm_eps", 1e-6), rope_theta=rp.get("rope_theta", 1e6),
                       tie_word_embeddings=tc.get("tie_word_embeddings", False), eos_token_ids=eos if isinstance(eos, list) else [eos],
                       partial_rotary_factor=rp.get("partial_rotary_factor", 1.0), attn_output_gate=tc.get("attn_output_gate", False),
                       layer_types=list(tc.get("layer_types", [])), linear_num_key_heads=tc.get("linear_num_key_heads", 16),
                       linear_key_head_dim=tc.get("linear_key_head_dim", 128), linear_num_value_heads=tc.get("linear_num_value_heads", 16),
                       linear_value_head_dim=tc.get("linear_value_head_dim", 128), linear_conv_kernel_dim=tc.get("linear_conv_kernel_dim", 4),
                       gemma_norm=True, weight_prefix="model.language_model.")
        eos = raw.get("eos_token_id", 151645)
        return cls(model_type="qwen3", hidden_size=raw["hidden_size"], intermediate_size=raw["intermediate_size"],
                   num_hidden_layers=raw["num_hidden_layers"], num_attention_heads=raw["num_attention_heads"],
                   num_key_value_heads=raw["num_key_value_heads"], head_dim=raw.get("head_dim", raw["hidden_size"] // raw["num_attention_heads"]),
                   vocab_size=raw["vocab_size"], rms_norm_eps=raw.get("rms_norm_eps", 1e-6), rope_theta=raw.get("rope_theta", 1e6),
                   tie_word_embeddings=raw.get("tie_word_embeddings", False), attention_bias=raw.get("attention_bias", False),
                   eos_token_ids=eos if isinstance(eos, list) else [eos])

    @classmethod
    def tiny(cls, hybrid: bool = False) -> "DenseConfig":
        if hybrid:
            return cls(model_type="qwen3_5", hidden_size=128, intermediate_size=256, num_hidden_layers=4, num_attention_heads=4,
                       num_key_value_heads=2, head_dim=64, vocab_size=512, partial_rotary_factor=0.5, attn_output_gate=True,
                       layer_types=["linear_attention", "linear_attention", "linear_attention", "full_attention"],
                       linear_num_key_heads=2, linear_key_head_dim=64, linear_num_value_heads=2, linear_value_head_dim=64,
                       gemma_norm=True, weight_prefix="model.language_model.", eos_token_ids=[1])
        return cls(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                   head_dim=64, vocab_size=512, eos_token_ids=[1])


@dataclass
class DenseLayer:
    kind: str
    input_norm: torch.Tensor
    post_attn_norm: torch.Tensor
    mlp_w13: LinearWeight                  # gate | up, rows [2 * I_local, H]
    mlp_w2: LinearWeight                   # [H, I_local]
    # full attention
    w_qkv: Optional[LinearWeight] = None   # q (| gate per head) | k | v rows
    q_norm: Optional[torch.Tensor] = None
    k_norm: Optional[torch.Tensor] = None
    o_proj: Optional[LinearWeight] = None
    # Gated DeltaNet
    w_in: Optional[LinearWeight] = None    # qkv | z | a | b rows
    conv_w: Optional[torch.Tensor] = None  # [conv_dim_local, Kw]
    A_log: Optional[torch.Tensor] = None
    dt_bias: Optional[torch.Tensor] = None
    gdn_norm: Optional[torch.Tensor] = None
    out_proj: Optional[LinearWeight] = None


@dataclass
class DenseWeights:
    embed: torch.Tensor
    layers: List[DenseLayer]
    final_norm: torch.Tensor
    lm_head: LinearWeight
    vocab_offset: int = 0


class DenseCache:
    """Paged bf16 K/V per full-attention layer; conv + recurrent state per linear-attention layer
    (indexed by a per-sequence state slot).  Reference: `PagedKVCache` dense layout and recurrent
    layers (`src/paged_kv.ts:82-106`, `Qwen35ChatCache`)."""

    def __init__(self, cfg: DenseConfig, num_pages: int, device, tp: int = 1, max_states: int = 64, dtype=torch.bfloat16):
        self.num_pages, self.page_size = num_pages, PAGE_SIZE
        n_kv = max(1, cfg.num_key_value_heads // tp)
        lh = max(1, cfg.linear_num_key_heads // tp)
        self.k, self.v, self.conv, self.rec = {}, {}, {}, {}
        for i, kind in enumerate(cfg.layer_types):
            if kind == "full_attention":
                self.k[i] = torch.zeros(num_pages * PAGE_SIZE, n_kv, cfg.head_dim, dtype=dtype, device=device)
                self.v[i] = torch.zeros_like(self.k[i])
            else:
                cdim = lh * (2 * cfg.linear_key_head_dim + cfg.linear_value_head_dim)
                self.conv[i] = torch.zeros(max_states, cdim, cfg.linear_conv_kernel_dim - 1, dtype=torch.float32, device=device)
                self.rec[i] = torch.zeros(max_states, lh, cfg.linear_key_head_dim, cfg.linear_value_head_dim, dtype=torch.float32,
                                          device=device)
        self.layers = list(range(len(cfg.layer_types)))
        self.max_states = max_states

    def copy_page(self, src: int, dst: int) -> None:
        a, b = slice(src * PAGE_SIZE, (src + 1) * PAGE_SIZE), slice(dst * PAGE_SIZE, (dst + 1) * PAGE_SIZE)
        for i in self.k:
            self.k[i][b] = self.k[i][a]
            self.v[i][b] = self.v[i][a]

    def page_tensors(self):
        """Slot-indexed tensors in a fixed order (host prefix tier); None for hybrid models, whose recurrent and
        convolution state belongs to a sequence, not to its pages."""
        if self.conv:
            return None
        return [t for i in sorted(self.k) for t in (self.k[i], self.v[i])]

    def reset_state(self, slot: int) -> None:
        for i in self.conv:
            self.conv[i][slot].zero_()
            self.rec[i][slot].zero_()

    def nbytes(self) -> int:
        t = list(self.k.values()) + list(self.v.values()) + list(self.conv.values()) + list(self.rec.values())
        return sum(x.numel() * x.element_size() for x in t)


class DenseModel:
    """Forward pass of the Qwen3 / Qwen3.5 decoders over the paged cache."""

    def __init__(self, cfg: DenseConfig, weights: DenseWeights, ctx: Optional[ParallelContext] = None, ops=None,
                 comm: Optional[Comm] = None):
        self.cfg, self.w = cfg, weights
        self.ctx = ctx or ParallelContext()
        self.ops = ops or get_ops(cfg, self.ctx.device, self.ctx)
        self.comm = comm or Comm(self.ctx)
        # linear-attention state needs one slot per live sequence; prefix sharing cannot restore it
        self.supports_prefix_sharing = "linear_attention" not in cfg.layer_types
        self._slot_of: Dict[int, int] = {}
        self._free_slots: List[int] = []
        self._state_idx: Optional[torch.Tensor] = None
        self._cache: Optional[DenseCache] = None

    # ---- engine hooks ----------------------------------------------------------------------------------
    def allocate_cache(self, num_pages: int, max_states: int = 64) -> DenseCache:
        self._cache = DenseCache(self.cfg, num_pages, self.ctx.device, self.ctx.world, max_states,
                                 dtype=torch.bfloat16 if self.ctx.device.type == "cuda" else torch.float32)
        self._free_slots = list(range(max_states - 1, -1, -1))
        self._state_idx = torch.zeros(max_states, dtype=torch.int32, device=self.ctx.device)
        return self._cache

    def prepare_step(self, st, seqs) -> None:
        """Host-side, outside any graph capture: give every sequence a recurrent-state slot (zeroed
        on first use) and upload the slot of each batch row."""
        if self.supports_prefix_sharing or self._cache is None:
            return
        slots = []
        for s in seqs:
            if s.seq_id not in self._slot_of:
                if not self._free_slots:
                    raise RuntimeError("out of recurrent-state slots")
                self._slot_of[s.seq_id] = self._free_slots.pop()
                self._cache.reset_state(self._slot_of[s.seq_id])
            slots.append(self._slot_of[s.seq_id])
        self._state_idx[: len(slots)].copy_(torch.tensor(slots, dtype=torch.int32), non_blocking=True)

    def release_sequence(self, seq_id: int) -> None:
        slot = self._slot_of.pop(seq_id, None)
        if slot is not None:
            self._free_slots.append(slot)

    # ---- layers -------------------------------------------------------------------------------------------
    def _qo_indptr(self, st):
        """Token ranges of the step's sequences: one token per page-table row in a decode step,
        otherwise one sequence holding every token (the engine prefills one sequence per chunk)."""
        q = st.extra.get("qo_indptr")
        if q is not None:
            return q, st.extra.get("max_q", st.num_tokens)
        T, B = st.num_tokens, st.page_table.shape[0]
        if T == B:
            return None, 1
        return torch.tensor([0, T], dtype=torch.int32, device=st.input_ids.device), T

    @traced(lambda self, i, *a, **k: f"layer{i}.attention")
    def _full_attention(self, i: int, lw: DenseLayer, x, st, cache: DenseCache):
        cfg, ops = self.cfg, self.ops
        T = x.shape[0]
        hl = lw.o_proj.in_features // cfg.head_dim
        kvl = cache.k[i].shape[1]
        qs = cfg.head_dim * (2 if cfg.attn_output_gate else 1)
        qkv = ops.linear(x, lw.w_qkv)
        q, k, v = qkv[:, :hl * qs], qkv[:, hl * qs:hl * qs + kvl * cfg.head_dim], qkv[:, hl * qs + kvl * cfg.head_dim:]
        q_out = D.qk_norm_rope_cache(q, k, v, lw.q_norm, lw.k_norm, st.positions, st.batch_idx, st.page_table, st.page_size,
                                     cache.k[i], cache.v[i], hl, kvl, cfg.head_dim, cfg.rope_dim, cfg.rope_theta,
                                     cfg.rms_norm_eps, q_stride=qs)
        qo, max_q = self._qo_indptr(st)
        o = D.paged_attention(q_out, cache.k[i], cache.v[i], st.positions, st.batch_idx, st.page_table, st.page_size,
                              cfg.scaling, qo_indptr=qo, max_q=max_q, max_kv_len=st.max_kv_len)
        if cfg.attn_output_gate:
            gate = q.reshape(T, hl, qs)[..., cfg.head_dim:]
            o = (o.to(torch.float32) * torch.sigmoid(gate.to(torch.float32))).to(o.dtype)
        return ops.linear(o.reshape(T, hl * cfg.head_dim), lw.o_proj, out_f32=True)

    @traced(lambda self, i, *a, **k: f"layer{i}.linear_attention")
    def _linear_attention(self, i: int, lw: DenseLayer, x, st, cache: DenseCache):
        cfg, ops = self.cfg, self.ops
        T = x.shape[0]
        dk, dv = cfg.linear_key_head_dim, cfg.linear_value_head_dim
        lh = cache.rec[i].shape[1]
        cdim, zdim = lh * (2 * dk + dv), lh * dv
        proj = ops.linear(x, lw.w_in)
        qkv, z, a, b = proj[:, :cdim], proj[:, cdim:cdim + zdim], proj[:, cdim + zdim:cdim + zdim + lh], proj[:, cdim + zdim + lh:]
        qo, _ = self._qo_indptr(st)
        if qo is None:
            qo = torch.arange(T + 1, dtype=torch.int32, device=x.device)
        sidx = self._state_idx if self._state_idx is not None else torch.zeros(qo.numel() - 1, dtype=torch.int32, device=x.device)
        conv = RC.causal_conv1d(qkv, lw.conv_w, None, cache.conv[i], qo, sidx, activation=True)
        o = RC.gdn_scan(conv, a.contiguous(), b.contiguous(), lw.A_log, lw.dt_bias, cache.rec[i], qo, sidx, lh, dk, dv)
        gated = RC.rmsnorm_gated(o.reshape(T * lh, dv), z.reshape(T * lh, dv), lw.gdn_norm, cfg.rms_norm_eps)
        return ops.linear(gated.reshape(T, zdim), lw.out_proj, out_f32=True)

    @traced("mlp")
    def _mlp(self, lw: DenseLayer, y):
        return self.ops.dense_mlp(y, lw)

    def forward_hidden(self, st, cache: DenseCache) -> torch.Tensor:
        ops, comm, cfg = self.ops, self.comm, self.cfg
        partial, residual = ops.embed(st.input_ids, self.w.embed), None
        x, residual = ops.add_rmsnorm(partial, residual, self.w.layers[0].input_norm, cfg.rms_norm_eps)
        for i, lw in enumerate(self.w.layers):
            attn = self._full_attention(i, lw, x, st, cache) if lw.kind == "full_attention" else self._linear_attention(i, lw, x, st, cache)
            y, residual = comm.allreduce_add_rmsnorm(ops, attn, residual, lw.post_attn_norm, cfg.rms_norm_eps)
            mlp = self._mlp(lw, y)
            nxt = self.w.layers[i + 1].input_norm if i + 1 < len(self.w.layers) else self.w.final_norm
            x, residual = comm.allreduce_add_rmsnorm(ops, mlp, residual, nxt, cfg.rms_norm_eps)
        return x

    def compute_logits(self, hidden: torch.Tensor) -> torch.Tensor:
        local = self.ops.logits(hidden, self.w.lm_head)
        if self.ctx.world == 1:
            return local
        return self.comm.all_gather(local, dim=-1)


# ---- weights: random init (tests, benchmarks) and HF safetensors loading ------------------------------------

FP8_LINEAR_DEFAULT = False      # keep FP8 checkpoints' projections in FP8 (True) or expand them to bf16 at load


def _lin(t: torch.Tensor) -> LinearWeight:
    return LinearWeight(t.contiguous())


def random_dense_model(cfg: DenseConfig, seed: int = 0, device="cpu", dtype=torch.bfloat16, rank: int = 0, world: int = 1) -> DenseWeights:
    """Random weights with the checkpoint's shapes, sharded for `rank` of `world`: the full
    matrices are drawn from the seed on every rank and sliced, so shards agree."""
    g = torch.Generator().manual_seed(seed)
    H, I, hd = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim
    tensors: Dict[str, torch.Tensor] = {}
    pfx = cfg.weight_prefix

    def rnd(*shape, scale=None):
        s = scale if scale is not None else shape[-1] ** -0.5
        return (torch.randn(*shape, generator=g) * s).to(torch.bfloat16)

    def norm_w(n):
        w = 1.0 + 0.1 * torch.randn(n, generator=g)
        return (w - 1.0 if cfg.gemma_norm else w).to(torch.bfloat16)

    tensors[pfx + "embed_tokens.weight"] = rnd(cfg.vocab_size, H, scale=1.0)
    for i, kind in enumerate(cfg.layer_types):
        lp = f"{pfx}layers.{i}."
        tensors[lp + "input_layernorm.weight"] = norm_w(H)
        tensors[lp + "post_attention_layernorm.weight"] = norm_w(H)
        tensors[lp + "mlp.gate_proj.weight"] = rnd(I, H)
        tensors[lp + "mlp.up_proj.weight"] = rnd(I, H)
        tensors[lp + "mlp.down_proj.weight"] = rnd(H, I)
        if kind == "full_attention":
            qs = hd * (2 if cfg.attn_output_gate else 1)
            tensors[lp + "self_attn.q_proj.weight"] = rnd(cfg.num_attention_heads * qs, H)
            tensors[lp + "self_attn.k_proj.weight"] = rnd(cfg.num_key_value_heads * hd, H)
            tensors[lp + "self_attn.v_proj.weight"] = rnd(cfg.num_key_value_heads * hd, H)
            tensors[lp + "self_attn.o_proj.weight"] = rnd(H, cfg.num_attention_heads * hd)
            tensors[lp + "self_attn.q_norm.weight"] = norm_w(hd)
            tensors[lp + "self_attn.k_norm.weight"] = norm_w(hd)
        else:
            lh, dk, dv, kw = cfg.linear_num_key_heads, cfg.linear_key_head_dim, cfg.linear_value_head_dim, cfg.linear_conv_kernel_dim
            tensors[lp + "linear_attn.in_proj_qkv.weight"] = rnd(cfg.conv_dim, H)
            tensors[lp + "linear_attn.in_proj_z.weight"] = rnd(lh * dv, H)
            tensors[lp + "linear_attn.in_proj_a.weight"] = rnd(lh, H)
            tensors[lp + "linear_attn.in_proj_b.weight"] = rnd(lh, H)
            tensors[lp + "linear_attn.conv1d.weight"] = rnd(cfg.conv_dim, 1, kw, scale=0.5)
            tensors[lp + "linear_attn.A_log"] = torch.log(torch.rand(lh, generator=g) * 2 + 0.5)
            tensors[lp + "linear_attn.dt_bias"] = torch.randn(lh, generator=g) * 0.1
            tensors[lp + "linear_attn.norm.weight"] = (1.0 + 0.1 * torch.randn(dv, generator=g)).to(torch.bfloat16)
            tensors[lp + "linear_attn.out_proj.weight"] = rnd(H, lh * dv)
    tensors[pfx + "norm.weight"] = norm_w(H)
    if not cfg.tie_word_embeddings:
        tensors["lm_head.weight"] = rnd(cfg.vocab_size, H)
    return assemble_dense_weights(cfg, tensors, device, dtype, rank, world), tensors


def _fp8_rows(w: LinearWeight, lo: int, hi: int) -> LinearWeight:
    if w.is_fp8 and (lo % 128 or (hi % 128 and hi != w.out_features)):
        w = LinearWeight(w.dequant(torch.bfloat16))             # shard edge inside a scale block: expand
    return w.rows(lo, hi)


def _fp8_cols(w: LinearWeight, lo: int, hi: int) -> LinearWeight:
    if w.is_fp8 and (lo % 128 or (hi % 128 and hi != w.in_features)):
        w = LinearWeight(w.dequant(torch.bfloat16))
    return w.cols(lo, hi)


def _fp8_cat(ws) -> LinearWeight:
    """Stack weights along the output features; stays FP8 when every part but the last ends on a scale-block edge."""
    if all(w.is_fp8 for w in ws) and all(w.out_features % 128 == 0 for w in ws[:-1]):
        w8 = torch.cat([w.weight.view(torch.uint8) for w in ws], 0).view(torch.float8_e4m3fn)
        return LinearWeight(w8, fp8_scale=torch.cat([w.fp8_scale for w in ws], 0))
    return LinearWeight(torch.cat([w.dequant(torch.bfloat16) if w.is_fp8 else w.weight for w in ws], 0))


def assemble_dense_weights(cfg: DenseConfig, tensors: Dict[str, torch.Tensor], device, dtype, rank: int = 0, world: int = 1,
                           keep_fp8: Optional[bool] = None) -> DenseWeights:
    """Checkpoint tensors (HF names) -> fused, TP-sharded runtime weights.  With `keep_fp8` (default: the
    `SLOPLLM_B200_FP8_LINEAR` switch) the FP8 block-quantised projections of attention and MLP stay in FP8 and are served by
    the FP8 kernels (`csrc/fp8_linear.cu`; reference `csrc/glm_gemv.cu:323-500`); otherwise they are expanded to `dtype` here."""
    from ..config import env_flag
    pfx, hd, H = cfg.weight_prefix, cfg.head_dim, cfg.hidden_size
    keep_fp8 = env_flag("FP8_LINEAR", FP8_LINEAR_DEFAULT) if keep_fp8 is None else keep_fp8

    def getw(name) -> LinearWeight:
        t = tensors[name]
        scale_name = name + "_scale_inv"
        if scale_name in tensors and keep_fp8:
            t8 = t.view(torch.float8_e4m3fn) if t.dtype == torch.uint8 else t
            return LinearWeight(t8, fp8_scale=tensors[scale_name].to(torch.float32))
        return LinearWeight(get(name))

    def wrows(w: LinearWeight, units: Optional[int] = None, per_unit: int = 1) -> LinearWeight:
        n = (w.out_features if units is None else units) // world
        return _fp8_rows(w, rank * n * per_unit, (rank + 1) * n * per_unit)

    def wcols(w: LinearWeight) -> LinearWeight:
        n = w.in_features // world
        return _fp8_cols(w, rank * n, (rank + 1) * n)

    def fin(w: LinearWeight) -> LinearWeight:
        return w.to(device, dtype)

    def get(name):
        t = tensors[name]
        scale_name = name + "_scale_inv"
        if scale_name in tensors:                       # FP8 block-quantised linear
            t = D.fp8_block_dequant(t, tensors[scale_name])
        return t

    def norm(name):
        w = tensors[name].to(torch.float32)
        return (w + 1.0 if cfg.gemma_norm else w).to(dtype).to(device)

    def rows(t, r=rank, w=world):
        n = t.shape[0] // w
        return t[r * n:(r + 1) * n]

    def cols(t, r=rank, w=world):
        n = t.shape[1] // w
        return t[:, r * n:(r + 1) * n]

    def head_rows(t, heads, per_head):
        return rows(t.reshape(heads, per_head, -1)).reshape(-1, t.shape[-1])

    dev = lambda t: t.to(dtype).to(device)
    layers = []
    for i, kind in enumerate(cfg.layer_types):
        lp = f"{pfx}layers.{i}."
        w13 = _fp8_cat([wrows(getw(lp + "mlp.gate_proj.weight")), wrows(getw(lp + "mlp.up_proj.weight"))])
        lw = DenseLayer(kind=kind, input_norm=norm(lp + "input_layernorm.weight"), post_attn_norm=norm(lp + "post_attention_layernorm.weight"),
                        mlp_w13=fin(w13), mlp_w2=fin(wcols(getw(lp + "mlp.down_proj.weight"))))
        if kind == "full_attention":
            qs = hd * (2 if cfg.attn_output_gate else 1)
            q = wrows(getw(lp + "self_attn.q_proj.weight"), cfg.num_attention_heads, qs)
            k = wrows(getw(lp + "self_attn.k_proj.weight"), cfg.num_key_value_heads, hd)
            v = wrows(getw(lp + "self_attn.v_proj.weight"), cfg.num_key_value_heads, hd)
            lw.w_qkv = fin(_fp8_cat([q, k, v]))
            lw.o_proj = fin(wcols(getw(lp + "self_attn.o_proj.weight")))
            lw.q_norm = norm(lp + "self_attn.q_norm.weight") if lp + "self_attn.q_norm.weight" in tensors else None
            lw.k_norm = norm(lp + "self_attn.k_norm.weight") if lp + "self_attn.k_norm.weight" in tensors else None
        else:
            lh, dk, dv = cfg.linear_num_key_heads, cfg.linear_key_head_dim, cfg.linear_value_head_dim
            qkv = get(lp + "linear_attn.in_proj_qkv.weight")
            conv = tensors[lp + "linear_attn.conv1d.weight"].reshape(cfg.conv_dim, -1)
            # q | k | v sections are sharded by head separately (`src/qwen35_model.ts:171-190`)
            secs = [(0, lh * dk, dk), (lh * dk, 2 * lh * dk, dk), (2 * lh * dk, 2 * lh * dk + lh * dv, dv)]
            qkv_l = torch.cat([head_rows(qkv[a:b], lh, d) for a, b, d in secs], 0)
            conv_l = torch.cat([head_rows(conv[a:b], lh, d) for a, b, d in secs], 0)
            z = head_rows(get(lp + "linear_attn.in_proj_z.weight"), lh, dv)
            a_w, b_w = rows(get(lp + "linear_attn.in_proj_a.weight")), rows(get(lp + "linear_attn.in_proj_b.weight"))
            lw.w_in = _lin(dev(torch.cat([qkv_l, z, a_w, b_w], 0)))
            lw.conv_w = dev(conv_l).contiguous()
            lw.A_log = rows(tensors[lp + "linear_attn.A_log"].to(torch.float32)).to(device).contiguous()
            lw.dt_bias = rows(tensors[lp + "linear_attn.dt_bias"].to(torch.float32)).to(device).contiguous()
            lw.gdn_norm = dev(tensors[lp + "linear_attn.norm.weight"])
            lw.out_proj = _lin(dev(cols(get(lp + "linear_attn.out_proj.weight"))))
        layers.append(lw)
    embed = dev(tensors[pfx + "embed_tokens.weight"])
    head = tensors["lm_head.weight"] if "lm_head.weight" in tensors else tensors[pfx + "embed_tokens.weight"]
    vloc = head.shape[0] // world
    return DenseWeights(embed=embed, layers=layers, final_norm=norm(pfx + "norm.weight"), lm_head=_lin(dev(rows(head))),
                        vocab_offset=rank * vloc)


def load_dense_model(model_dir: str, ctx: Optional[ParallelContext] = None, dtype=torch.bfloat16):
    """(cfg, DenseModel) from a HF directory of safetensors shards (text decoder only: `model.visual.*` is skipped)."""
    from ..checkpoint.safetensors_io import SafetensorsFile
    ctx = ctx or ParallelContext()
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = DenseConfig.from_hf_dict(json.load(f))
    tensors: Dict[str, torch.Tensor] = {}
    for fn in sorted(os.listdir(model_dir)):
        if fn.endswith(".safetensors"):
            sf = SafetensorsFile(os.path.join(model_dir, fn))
            for name in sf.names():
                if not name.startswith("model.visual."):
                    tensors[name] = sf.tensor(name)
    w = assemble_dense_weights(cfg, tensors, ctx.device, dtype, ctx.rank if ctx.world > 1 else 0, ctx.world)
    return cfg, DenseModel(cfg, w, ctx)
