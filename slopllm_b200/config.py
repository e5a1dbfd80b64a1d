"""Typed configuration: model architecture, engine/runtime knobs, environment switches.

Parity: the reference parses `config.json` in `src/glm51_model.ts:95-147` (glm_moe_dsa),
its CLI flags in `src/openai-server.ts:51-103` / `src/model_cli.ts:1-154`, and ~35
`SLOPLLM_*` environment switches read at module load.  Here all three live in
dataclasses; environment overrides use the single prefix `SLOPLLM_B200_`.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, asdict
from typing import List, Optional

PAGE_SIZE = 64  # tokens per KV page (reference: src/paged_sequence.ts PAGE_SIZE)


def env_flag(name: str, default: bool = False) -> bool:
    v = os.environ.get("SLOPLLM_B200_" + name)
    if v is None:
        return default
    return v.strip().lower() not in ("0", "false", "no", "off", "")


def env_int(name: str, default: int) -> int:
    v = os.environ.get("SLOPLLM_B200_" + name)
    return default if v is None or v == "" else int(v)


def env_str(name: str, default: str = "") -> str:
    return os.environ.get("SLOPLLM_B200_" + name, default)


@dataclass
class GlmMoeDsaConfig:
    """Architecture of the glm_moe_dsa family (MLA + DSA indexer + sigmoid MoE + MTP)."""

    hidden_size: int = 6144
    intermediate_size: int = 12288          # dense MLP layers
    moe_intermediate_size: int = 2048
    num_hidden_layers: int = 78
    num_nextn_predict_layers: int = 1       # MTP layers appended after the stack
    rms_norm_eps: float = 1e-5
    vocab_size: int = 154880
    tie_word_embeddings: bool = False
    num_attention_heads: int = 64
    q_lora_rank: int = 2048
    kv_lora_rank: int = 512
    qk_nope_head_dim: int = 192
    qk_rope_head_dim: int = 64
    v_head_dim: int = 256
    rope_theta: float = 1e6
    rope_interleave: bool = True
    indexer_rope_interleave: bool = True
    n_routed_experts: int = 256
    n_shared_experts: int = 1
    num_experts_per_tok: int = 8
    n_group: int = 1
    topk_group: int = 1
    norm_topk_prob: bool = True
    routed_scaling_factor: float = 2.5
    index_topk: int = 2048
    index_head_dim: int = 128
    index_n_heads: int = 32
    indexer_types: Optional[List[str]] = None     # "full" | "shared" per layer (+ MTP)
    index_share_for_mtp_iteration: bool = False
    mlp_layer_types: Optional[List[str]] = None   # "dense" | "sparse"
    first_k_dense_replace: int = 3
    eos_token_ids: List[int] = field(default_factory=lambda: [2])
    # Which linear layers are NVFP4 in a synthetic / quantised checkpoint.  The real
    # GLM-5 NVFP4 checkpoint quantises only routed + shared experts; the benchmark
    # configuration additionally quantises o_proj and the dense MLP.
    quant_experts: bool = True
    quant_o_proj: bool = False
    quant_dense_mlp: bool = False

    def __post_init__(self) -> None:
        n = self.num_hidden_layers
        if self.mlp_layer_types is None:
            k = min(self.first_k_dense_replace, n)
            self.mlp_layer_types = ["dense"] * k + ["sparse"] * (n - k)
        total = n + self.num_nextn_predict_layers
        if self.indexer_types is None:
            self.indexer_types = ["full"] * total
        elif len(self.indexer_types) == n and self.num_nextn_predict_layers:
            tail = "shared" if self.index_share_for_mtp_iteration else "full"
            self.indexer_types = list(self.indexer_types) + [tail] * self.num_nextn_predict_layers
        if self.n_routed_experts and self.n_group > 1:
            assert self.n_routed_experts % self.n_group == 0

    # ---- derived -------------------------------------------------------------------
    @property
    def qk_head_dim(self) -> int:
        return self.qk_nope_head_dim + self.qk_rope_head_dim

    @property
    def softmax_scale(self) -> float:
        return float(self.qk_head_dim) ** -0.5

    @property
    def kv_quant_group(self) -> int:
        """Values per fp8 scale in the packed cache row (128; the whole latent if smaller)."""
        return 128 if self.kv_lora_rank % 128 == 0 else self.kv_lora_rank

    @property
    def kv_row_bytes(self) -> int:
        """Packed sparse-MLA cache row: fp8 ckv + one f32 scale per group + bf16 rope."""
        g = self.kv_quant_group
        return self.kv_lora_rank + (self.kv_lora_rank // g) * 4 + self.qk_rope_head_dim * 2

    @property
    def index_row_bytes(self) -> int:
        return self.index_head_dim + 4

    def is_moe_layer(self, layer: int) -> bool:
        if layer >= self.num_hidden_layers:       # MTP layers follow the last layer's type
            return self.n_routed_experts > 0
        return self.mlp_layer_types[layer] == "sparse"

    def indexer_is_full(self, layer: int) -> bool:
        return self.indexer_types[layer] == "full"

    # ---- (de)serialisation -----------------------------------------------------------
    @classmethod
    def from_hf_dict(cls, raw: dict) -> "GlmMoeDsaConfig":
        n = raw["num_hidden_layers"]
        nope = raw.get("qk_nope_head_dim", 0)
        rope = raw.get("qk_rope_head_dim", 0)
        rp = raw.get("rope_parameters") or {}
        eos = raw.get("eos_token_id", 2)
        return cls(
            hidden_size=raw["hidden_size"],
            intermediate_size=raw["intermediate_size"],
            moe_intermediate_size=raw.get("moe_intermediate_size", raw["intermediate_size"]),
            num_hidden_layers=n,
            num_nextn_predict_layers=raw.get("num_nextn_predict_layers", 0) or 0,
            rms_norm_eps=raw.get("rms_norm_eps", 1e-5),
            vocab_size=raw["vocab_size"],
            tie_word_embeddings=raw.get("tie_word_embeddings", False),
            num_attention_heads=raw["num_attention_heads"],
            q_lora_rank=raw["q_lora_rank"],
            kv_lora_rank=raw["kv_lora_rank"],
            qk_nope_head_dim=nope,
            qk_rope_head_dim=rope,
            v_head_dim=raw.get("v_head_dim", 0),
            rope_theta=rp.get("rope_theta", raw.get("rope_theta", 1e6)),
            rope_interleave=raw.get("rope_interleave", False),
            indexer_rope_interleave=raw.get("indexer_rope_interleave", raw.get("rope_interleave", False)),
            n_routed_experts=raw.get("n_routed_experts", 0),
            n_shared_experts=raw.get("n_shared_experts", 0),
            num_experts_per_tok=raw.get("num_experts_per_tok", raw.get("topk", 4)),
            n_group=raw.get("n_group", 1),
            topk_group=raw.get("topk_group", 1),
            norm_topk_prob=raw.get("norm_topk_prob", False),
            routed_scaling_factor=raw.get("routed_scaling_factor", 1.0),
            index_topk=raw.get("index_topk", 256),
            index_head_dim=raw.get("index_head_dim", 64),
            index_n_heads=raw.get("index_n_heads", 4),
            indexer_types=raw.get("indexer_types"),
            index_share_for_mtp_iteration=raw.get("index_share_for_mtp_iteration", False),
            mlp_layer_types=raw.get("mlp_layer_types", None) and list(raw["mlp_layer_types"])[:n],
            first_k_dense_replace=raw.get("first_k_dense_replace", 3),
            eos_token_ids=list(eos) if isinstance(eos, (list, tuple)) else [eos],
            quant_experts=raw.get("quant_experts", True),
            quant_o_proj=raw.get("quant_o_proj", False),
            quant_dense_mlp=raw.get("quant_dense_mlp", False),
        )

    @classmethod
    def from_pretrained(cls, model_dir: str) -> "GlmMoeDsaConfig":
        with open(os.path.join(model_dir, "config.json")) as f:
            return cls.from_hf_dict(json.load(f))

    def to_hf_dict(self) -> dict:
        d = asdict(self)
        d["model_type"] = "glm_moe_dsa"
        d["eos_token_id"] = d.pop("eos_token_ids")
        d["indexer_types"] = self.indexer_types[: self.num_hidden_layers]
        d["rope_parameters"] = {"rope_theta": self.rope_theta, "rope_type": "default"}
        return d

    # ---- named configurations ----------------------------------------------------------
    @classmethod
    def tiny(cls) -> "GlmMoeDsaConfig":
        """The CPU plumbing model: 2 layers (dense + MoE), hidden 256, vocab 1024."""
        return cls(
            hidden_size=256, intermediate_size=512, moe_intermediate_size=128,
            num_hidden_layers=2, num_nextn_predict_layers=1, vocab_size=1024,
            num_attention_heads=4, q_lora_rank=128, kv_lora_rank=64,
            qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32,
            n_routed_experts=8, n_shared_experts=1, num_experts_per_tok=2,
            n_group=1, topk_group=1, index_topk=64, index_head_dim=32, index_n_heads=2,
            first_k_dense_replace=1, eos_token_ids=[1023],
        )

    @classmethod
    def glm5(cls, num_layers: int = 78, quant_all: bool = True) -> "GlmMoeDsaConfig":
        """GLM-5-class shape (78 layers, hidden 6144, 256 experts, 8 routing groups)."""
        types = ["full" if (i < 3 or (i - 3) % 4 == 0) else "shared" for i in range(num_layers)]
        return cls(
            num_hidden_layers=num_layers, n_group=8, topk_group=4,
            indexer_types=types, index_share_for_mtp_iteration=False,
            first_k_dense_replace=min(3, num_layers),
            quant_o_proj=quant_all, quant_dense_mlp=quant_all,
            eos_token_ids=[154820, 154827, 154829],
        )


@dataclass
class SamplingParams:
    """Per-request sampling parameters (reference: src/chat_model.ts:24-31)."""

    temperature: float = 0.6
    top_p: float = 0.95
    top_k: int = 20
    repetition_penalty: float = 1.0
    presence_penalty: float = 0.0
    repetition_penalty_window: int = 64

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0 or self.top_k == 1


@dataclass
class EngineConfig:
    """Runtime knobs; field names follow the reference's CLI flags."""

    model: str = ""
    gpus: List[int] = field(default_factory=lambda: [0])
    arena_gb: float = 0.0              # 0: no cap on this process's device allocations
    cp: bool = False
    ep: bool = False                   # expert-parallel MoE instead of TP-sliced experts
    mtp: int = 0                       # number of draft tokens (0 = off; bare --mtp = 3)
    batch_size: int = 8
    chunk_size: int = 8192
    max_pages: int = 0                 # 0 => batch_size * ceil(chunk_size / 64)
    max_host_pages: int = 0
    phased_prefill: bool = True
    cuda_graph: bool = True
    max_tokens: int = 65536
    sampling: SamplingParams = field(default_factory=SamplingParams)
    decode_latency_ms: float = 0.0
    host: str = "127.0.0.1"
    port: int = 8000
    api_key: Optional[str] = None
    admin_api_key: Optional[str] = None
    fused_collectives: bool = True     # in-kernel NVLink collectives (else NCCL); `make_comm` also honours SLOPLLM_B200_FUSED=0

    def __post_init__(self) -> None:
        if self.max_pages <= 0:
            self.max_pages = self.batch_size * -(-self.chunk_size // PAGE_SIZE)
        n = len(self.gpus)
        if n & (n - 1):
            raise ValueError("--gpus needs a power-of-two device count")
