"""glm5_next scaffolding: config checks, tensor-parallel rules, the KDA sub-layer (prefill in one
go equals prefill + decode steps through the rolling state) and mHC shape checks.
Reference behaviour: `src/glm53_flash_model.ts`, `src/kda.ts`, `src/flash_hybrid_validation.ts`."""
import copy

import pytest
import torch

from slopllm_b200.models.glm5_next import (Glm5NextConfig, Glm5NextModel, KdaState, KdaWeights, kda_attention,
                                           weight_parallelism)
from slopllm_b200.ops import recurrent as RC

RAW = {"model_type": "glm5_next", "text_config": {
    "hidden_size": 256, "intermediate_size": 512, "num_hidden_layers": 3, "vocab_size": 1000, "num_attention_heads": 4,
    "num_key_value_heads": 4, "q_lora_rank": 64, "kv_lora_rank": 64, "qk_nope_head_dim": 64, "qk_rope_head_dim": 0, "v_head_dim": 64,
    "linear_attn_config": {"num_heads": 2, "head_dim": 128, "short_conv_kernel_size": 4, "gate_lower_bound": -5},
    "hc_mult": 4, "hc_eps": 1e-6, "hc_sinkhorn_iters": 20, "n_routed_experts": 8, "n_shared_experts": 1, "num_experts_per_tok": 2,
    "moe_intermediate_size": 128, "index_head_dim": 64, "index_n_heads": 4, "index_kpool": 4,
    "layer_types": ["linear_attention", "deepseek_sparse_attention", "indexed_attention"], "eos_token_id": 2}}


def test_config_validation():
    cfg = Glm5NextConfig.from_hf_dict(RAW)
    assert cfg.linear_num_heads == 2 and cfg.eos_token_ids == [2]
    bad = copy.deepcopy(RAW)
    bad["text_config"]["hc_mult"] = 2
    with pytest.raises(ValueError, match="geometry"):
        Glm5NextConfig.from_hf_dict(bad)
    bad = copy.deepcopy(RAW)
    bad["text_config"]["layer_types"][1] = "full_attention"
    with pytest.raises(ValueError, match="layer_types"):
        Glm5NextConfig.from_hf_dict(bad)
    bad = copy.deepcopy(RAW)
    bad["text_config"]["index_kpool"] = 0
    with pytest.raises(ValueError, match="index_kpool"):
        Glm5NextConfig.from_hf_dict(bad)
    with pytest.raises(ValueError, match="text_config"):
        Glm5NextConfig.from_hf_dict({"model_type": "glm5_next"})


def test_weight_parallelism_and_loader_rules():
    p = "model.language_model.layers.0."
    assert weight_parallelism(p + "self_attn.q_proj.weight") == "column"
    assert weight_parallelism(p + "self_attn.k_conv1d.weight") == "column"
    assert weight_parallelism(p + "self_attn.A_log") == "column"
    assert weight_parallelism(p + "self_attn.o_proj.weight") == "row"
    assert weight_parallelism(p + "mlp.experts.3.down_proj.weight_scale") == "row"
    assert weight_parallelism(p + "mlp.shared_experts.up_proj.weight") == "column"
    assert weight_parallelism(p + "self_attn.f_a_proj.weight") == "replicated"
    assert weight_parallelism("lm_head.weight") == "column"
    m = Glm5NextModel(Glm5NextConfig.from_hf_dict(RAW))
    m.load_tensor("model.visual.patch.weight", torch.zeros(2, 2))
    m.load_tensor("model.language_model.layers.7.mlp.gate.weight", torch.zeros(2, 2))       # MTP layer: skipped
    assert not m.tensors
    with pytest.raises(ValueError, match="unsupported"):
        m.load_tensor("something.else", torch.zeros(1))
    with pytest.raises(ValueError, match="BF16 linears"):
        m.load_tensor(p + "self_attn.q_proj.weight", torch.zeros(2, 2), "F8_E4M3")
    with pytest.raises(NotImplementedError):
        m.forward_hidden(None, None)
    with pytest.raises(ValueError, match="not KDA"):
        m.kda_weights(1)


def _weights(H, heads, g):
    W = heads * 128
    r = lambda *s: torch.randn(*s, generator=g) * s[-1] ** -0.5
    return KdaWeights(q=r(W, H), k=r(W, H), v=r(W, H), q_conv=r(W, 1, 4), k_conv=r(W, 1, 4), v_conv=r(W, 1, 4), f_a=r(32, H), f_b=r(W, 32),
                      beta=r(heads, H), g_a=r(32, H), g_b=r(W, 32), norm=torch.ones(128), out=r(H, W),
                      a_log=torch.zeros(heads), dt_bias=torch.zeros(W))


def test_kda_attention_resumes_from_state():
    g = torch.Generator().manual_seed(0)
    H, heads, T = 64, 2, 12
    w = _weights(H, heads, g)
    x = torch.randn(T, H, generator=g)
    sidx = torch.tensor([0], dtype=torch.int32)
    full_state = KdaState(1, heads, "cpu")
    full = kda_attention(x, w, full_state, torch.tensor([0, T], dtype=torch.int32), sidx)
    st = KdaState(1, heads, "cpu")
    a = kda_attention(x[:8], w, st, torch.tensor([0, 8], dtype=torch.int32), sidx)
    rest = [kda_attention(x[i:i + 1], w, st, torch.tensor([0, 1], dtype=torch.int32), sidx) for i in range(8, T)]
    got = torch.cat([a] + rest)
    assert full.shape == (T, H)
    assert (got - full).abs().max() / full.abs().max() < 2e-2
    assert (st.recurrent - full_state.recurrent).abs().max() < 1e-2
    with pytest.raises(ValueError, match="heads divisible"):
        KdaState(1, 3, "cpu", world=2)


def test_mhc_argument_checks():
    x = torch.zeros(2, 4, 8)
    with pytest.raises(ValueError):
        RC.mhc_pre(torch.zeros(2, 3, 8), torch.zeros(24, 32), torch.zeros(24), torch.zeros(3), 1e-6, 1e-6, 20)
    with pytest.raises(ValueError):
        RC.mhc_pre(x, torch.zeros(24, 16), torch.zeros(24), torch.zeros(3), 1e-6, 1e-6, 20)
    with pytest.raises(ValueError):
        RC.mhc_streams(x, True)
    assert RC.mhc_streams(torch.ones(2, 8), True).shape == (2, 4, 8)
