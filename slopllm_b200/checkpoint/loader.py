"""glm_moe_dsa checkpoint <-> ModelWeights.

Loading follows `src/chat_model.ts:602-699` (iterate the checkpoint source, shard every tensor
for this TP rank while it is still a host mapping, upload) and `src/glm51_model.ts:178-343`
(per-weight TP rule; kv_b_proj split into the absorbed `k_nope` [h, Dn, R] and `v_proj`
[h, R, Dv]; F32 norms -> activation dtype; `input_scale` discarded, `weight_scale_2` kept).
Replaced CSF scale tensors are decoded on the GPU (`sl_csf_decode`) when a device is given,
with the TP window applied by the decoder.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Optional

import torch

from ..config import GlmMoeDsaConfig
from ..models.weights import ExpertWeights, LayerWeights, LinearWeight, ModelWeights
from .safetensors_io import save_file
from .source import CheckpointSource, open_checkpoint_source


class _Reader:
    def __init__(self, src: CheckpointSource, device, dtype):
        self.src, self.device, self.dtype = src, torch.device(device), dtype

    def has(self, name: str) -> bool:
        return self.src.has(name)

    def _window(self, name: str, rows=None, cols=None) -> torch.Tensor:
        """This rank's window of a stored tensor as a contiguous host tensor: cut out of the mapping by the C++ runtime
        (threads, pinned destination for a GPU load) when it can, else a slice of the mapped tensor."""
        w = self.src.window(name, rows, cols, pin=self.device.type == "cuda") if hasattr(self.src, "window") else None
        if w is not None:
            return w
        t = self.src.tensor(name)
        if rows is not None:
            t = t[rows[0]:rows[1]]
        if cols is not None:
            t = t[:, cols[0]:cols[1]]
        return t

    def dense(self, name: str, rows=None, cols=None, dtype=None) -> torch.Tensor:
        t = self._window(name, rows, cols)
        dt = self.dtype if dtype is None else dtype
        return t.to(device=self.device, dtype=dt).contiguous()

    def scale(self, name: str, rows=None, cols=None) -> torch.Tensor:
        """E4M3 block-scale tensor; CSF planes are expanded by the GPU decoder when possible."""
        planes = self.src.csf_planes(name)
        if planes is not None and self.device.type == "cuda":
            from .csf_gpu import decode_csf_scales
            fixed, exc, (R, Cn) = planes
            r0, r1 = rows or (0, R)
            c0, c1 = cols or (0, Cn)
            return decode_csf_scales(fixed, exc, R, Cn, r0, r1 - r0, c0, c1 - c0, self.device)
        return self._window(name, rows, cols).contiguous().to(self.device)

    def linear(self, prefix: str, rows=None, cols=None) -> LinearWeight:
        """Linear `prefix.weight` (+ NVFP4 aux tensors).  rows / cols are in logical elements."""
        if self.has(prefix + ".weight_scale"):
            pc = None if cols is None else (cols[0] // 2, cols[1] // 2)
            sc = None if cols is None else (cols[0] // 16, cols[1] // 16)
            w = self._window(prefix + ".weight", rows, pc)
            g = self.src.tensor(prefix + ".weight_scale_2").to(torch.float32).reshape(()) if self.has(prefix + ".weight_scale_2") \
                else torch.ones(())
            return LinearWeight(w.contiguous().to(self.device), self.scale(prefix + ".weight_scale", rows, sc), g.to(self.device))
        return LinearWeight(self.dense(prefix + ".weight", rows, cols))


def load_config(model_dir: str) -> GlmMoeDsaConfig:
    src_dir = os.path.join(model_dir, "metadata") if os.path.exists(os.path.join(model_dir, "build-contract.json")) else model_dir
    with open(os.path.join(src_dir, "config.json")) as f:
        return GlmMoeDsaConfig.from_hf_dict(json.load(f))


def _experts(rd: _Reader, prefix: str, n: int, lo: int, hi: int, tp_rows, I: int) -> ExpertWeights:
    """Stack experts [lo, hi) of `prefix.{e}`; `tp_rows` = (i0, i1) slice of the intermediate dim."""
    i0, i1 = tp_rows
    w13, s13, g13, w2, s2, g2 = [], [], [], [], [], []
    quant = rd.has((f"{prefix}.{lo}" if n else prefix) + ".gate_proj.weight_scale")
    for e in range(lo, hi):
        p = f"{prefix}.{e}" if n else prefix
        gate = rd.linear(p + ".gate_proj", rows=(i0, i1))
        up = rd.linear(p + ".up_proj", rows=(i0, i1))
        down = rd.linear(p + ".down_proj", cols=(i0, i1))
        w13.append(torch.cat([gate.weight, up.weight]))
        w2.append(down.weight)
        if quant:
            s13.append(torch.cat([gate.scale, up.scale]))
            s2.append(down.scale)
            g13.append(torch.stack([gate.scale2.reshape(()), up.scale2.reshape(())]))
            g2.append(down.scale2.reshape(()))
    if quant:
        return ExpertWeights(torch.stack(w13), torch.stack(w2), torch.stack(s13), torch.stack(s2), torch.stack(g13).float(),
                             torch.stack(g2).float(), expert_offset=lo if n else 0)
    return ExpertWeights(torch.stack(w13), torch.stack(w2), expert_offset=lo if n else 0)


def load_layer(rd: _Reader, cfg: GlmMoeDsaConfig, layer: int, tp_rank: int, tp_world: int, ep: bool) -> LayerWeights:
    W, r = tp_world, tp_rank
    p = f"model.layers.{layer}"
    a = p + ".self_attn"
    h, hl = cfg.num_attention_heads, cfg.num_attention_heads // W
    Dn, Dr, Dv, R = cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim, cfg.kv_lora_rank
    full = cfg.indexer_is_full(layer) and rd.has(a + ".indexer.wq_b.weight")
    parts = [rd.dense(a + ".q_a_proj.weight"), rd.dense(a + ".kv_a_proj_with_mqa.weight")]
    qb = rd.dense(a + ".q_b_proj.weight", rows=(r * hl * (Dn + Dr), (r + 1) * hl * (Dn + Dr)))
    if full:
        parts += [rd.dense(a + ".indexer.wk.weight"), rd.dense(a + ".indexer.weights_proj.weight")]
        qb = torch.cat([qb, rd.dense(a + ".indexer.wq_b.weight")])
    kvb = rd.dense(a + ".kv_b_proj.weight", rows=(r * hl * (Dn + Dv), (r + 1) * hl * (Dn + Dv))).reshape(hl, Dn + Dv, R)
    lw = LayerWeights(
        input_norm=rd.dense(p + ".input_layernorm.weight"), post_attn_norm=rd.dense(p + ".post_attention_layernorm.weight"),
        w_qkv_a=LinearWeight(torch.cat(parts)), q_a_norm=rd.dense(a + ".q_a_layernorm.weight"),
        kv_a_norm=rd.dense(a + ".kv_a_layernorm.weight"), w_q_b=LinearWeight(qb.contiguous()),
        w_kn=kvb[:, :Dn, :].contiguous(), w_v=kvb[:, Dn:, :].transpose(1, 2).contiguous(),
        o_proj=rd.linear(a + ".o_proj", cols=(r * hl * Dv, (r + 1) * hl * Dv)), has_indexer=full,
        idx_k_norm_w=rd.dense(a + ".indexer.k_norm.weight") if full else None,
        idx_k_norm_b=rd.dense(a + ".indexer.k_norm.bias") if full else None)
    m = p + ".mlp"
    if rd.has(m + ".gate.weight"):
        E, I = cfg.n_routed_experts, cfg.moe_intermediate_size
        lw.router_w = rd.dense(m + ".gate.weight")
        lw.router_bias = rd.dense(m + ".gate.e_score_correction_bias", dtype=torch.float32) if rd.has(m + ".gate.e_score_correction_bias") \
            else torch.zeros(E, dtype=torch.float32, device=rd.device)
        Ir = I // W
        if ep and W > 1:
            per = E // W
            lw.experts = _experts(rd, m + ".experts", E, r * per, (r + 1) * per, (0, I), I)
        else:
            lw.experts = _experts(rd, m + ".experts", E, 0, E, (r * Ir, (r + 1) * Ir), I)
        if rd.has(m + ".shared_experts.gate_proj.weight"):
            Is = I * cfg.n_shared_experts
            lw.shared = _experts(rd, m + ".shared_experts", 0, 0, 1, (r * Is // W, (r + 1) * Is // W), Is)
    else:
        I = cfg.intermediate_size
        Ir = I // W
        gate = rd.linear(m + ".gate_proj", rows=(r * Ir, (r + 1) * Ir))
        up = rd.linear(m + ".up_proj", rows=(r * Ir, (r + 1) * Ir))
        if gate.is_nvfp4:
            # one global scale per fused weight: fold the ratio into the up half's block scales is lossy,
            # so keep both halves on the gate's global scale only when they agree
            if float(gate.scale2) != float(up.scale2):
                raise ValueError(f"{m}: gate_proj and up_proj use different NVFP4 global scales; cannot fuse")
        lw.mlp_w13 = LinearWeight.cat([gate, up])
        lw.mlp_w2 = rd.linear(m + ".down_proj", cols=(r * Ir, (r + 1) * Ir))
    if rd.has(p + ".eh_proj.weight"):
        lw.eh_proj = LinearWeight(rd.dense(p + ".eh_proj.weight"))
        lw.enorm, lw.hnorm = rd.dense(p + ".enorm.weight"), rd.dense(p + ".hnorm.weight")
        lw.shared_head_norm = rd.dense(p + ".shared_head.norm.weight")
    return lw


def load_model(model_dir: str, device="cpu", dtype=torch.float32, tp_rank: int = 0, tp_world: int = 1, ep: bool = False,
               with_mtp: bool = True, cfg: Optional[GlmMoeDsaConfig] = None):
    """Returns (cfg, ModelWeights) sharded for (tp_rank, tp_world)."""
    cfg = cfg or load_config(model_dir)
    src = open_checkpoint_source(model_dir)
    rd = _Reader(src, device, dtype)
    V = cfg.vocab_size
    Vr = V // tp_world
    embed = rd.dense("model.embed_tokens.weight")
    head_name = "lm_head.weight" if rd.has("lm_head.weight") else "model.embed_tokens.weight"
    lm = rd.dense(head_name, rows=(tp_rank * Vr, (tp_rank + 1) * Vr))
    n = cfg.num_hidden_layers + (cfg.num_nextn_predict_layers if with_mtp else 0)
    present = []
    for i in range(n):
        if not rd.has(f"model.layers.{i}.input_layernorm.weight"):
            break
        present.append(i)
    # Layers are read by a small pool of threads (`SLOPLLM_B200_LOAD_BATCH_SIZE`, default 8, as the reference's
    # `SLOPLLM_LOAD_BATCH_SIZE`, `src/chat_model.ts:602-699`): paging the mmap'd shards in and cutting this rank's strided
    # windows out of them overlaps with the uploads of the layers that are already in host memory.  A CSF container opens
    # its shards lazily, so it is read by one thread.
    from ..config import env_int
    workers = max(1, min(env_int("LOAD_BATCH_SIZE", 8), len(present)))
    if workers > 1 and src.csf is None:
        from concurrent.futures import ThreadPoolExecutor
        with ThreadPoolExecutor(max_workers=workers, thread_name_prefix="load") as pool:
            layers = list(pool.map(lambda i: load_layer(rd, cfg, i, tp_rank, tp_world, ep), present))
    else:
        layers = [load_layer(rd, cfg, i, tp_rank, tp_world, ep) for i in present]
    w = ModelWeights(embed=embed, layers=layers, final_norm=rd.dense("model.norm.weight"), lm_head=LinearWeight(lm),
                     vocab_offset=tp_rank * Vr)
    if src.csf is not None and rd.device.type == "cuda":
        from .csf_gpu import check_decode_status
        check_decode_status(rd.device)
    src.close()
    return cfg, w


# ---- saving (tests, synthetic checkpoints) ------------------------------------------------------------------


def _put_linear(out: Dict[str, torch.Tensor], prefix: str, lw: LinearWeight) -> None:
    out[prefix + ".weight"] = lw.weight.cpu()
    if lw.is_nvfp4:
        out[prefix + ".weight_scale"] = lw.scale.cpu()
        out[prefix + ".weight_scale_2"] = lw.scale2.cpu().reshape(())
        out[prefix + ".input_scale"] = torch.ones(())


def _put_experts(out, prefix: str, ex: ExpertWeights, numbered: bool) -> None:
    I = ex.inter
    for e in range(ex.num_experts):
        p = f"{prefix}.{e}" if numbered else prefix
        if ex.is_nvfp4:
            _put_linear(out, p + ".gate_proj", LinearWeight(ex.w13[e, :I], ex.s13[e, :I], ex.g13[e, 0]))
            _put_linear(out, p + ".up_proj", LinearWeight(ex.w13[e, I:], ex.s13[e, I:], ex.g13[e, 1]))
            _put_linear(out, p + ".down_proj", LinearWeight(ex.w2[e], ex.s2[e], ex.g2[e]))
        else:
            _put_linear(out, p + ".gate_proj", LinearWeight(ex.w13[e, :I]))
            _put_linear(out, p + ".up_proj", LinearWeight(ex.w13[e, I:]))
            _put_linear(out, p + ".down_proj", LinearWeight(ex.w2[e]))


def save_model(cfg: GlmMoeDsaConfig, w: ModelWeights, out_dir: str, dtype=torch.bfloat16) -> str:
    """Write an un-sharded (TP=1) model in the Hugging Face tensor naming."""
    os.makedirs(out_dir, exist_ok=True)
    t: Dict[str, torch.Tensor] = {"model.embed_tokens.weight": w.embed.cpu().to(dtype), "lm_head.weight": w.lm_head.weight.cpu().to(dtype),
                                  "model.norm.weight": w.final_norm.cpu().to(dtype)}
    Dn, Dr, Dv, R = cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim, cfg.kv_lora_rank
    h = cfg.num_attention_heads
    for i, lw in enumerate(w.layers):
        p, a, m = f"model.layers.{i}", f"model.layers.{i}.self_attn", f"model.layers.{i}.mlp"
        c = lambda x: x.cpu().to(dtype)
        t[p + ".input_layernorm.weight"], t[p + ".post_attention_layernorm.weight"] = c(lw.input_norm), c(lw.post_attn_norm)
        qkv = lw.w_qkv_a.weight
        q0, q1 = cfg.q_lora_rank, cfg.q_lora_rank + R + Dr
        t[a + ".q_a_proj.weight"], t[a + ".kv_a_proj_with_mqa.weight"] = c(qkv[:q0]), c(qkv[q0:q1])
        t[a + ".q_a_layernorm.weight"], t[a + ".kv_a_layernorm.weight"] = c(lw.q_a_norm), c(lw.kv_a_norm)
        qb = lw.w_q_b.weight
        t[a + ".q_b_proj.weight"] = c(qb[: h * (Dn + Dr)])
        if lw.has_indexer:
            t[a + ".indexer.wk.weight"] = c(qkv[q1:q1 + cfg.index_head_dim])
            t[a + ".indexer.weights_proj.weight"] = c(qkv[q1 + cfg.index_head_dim:])
            t[a + ".indexer.wq_b.weight"] = c(qb[h * (Dn + Dr):])
            t[a + ".indexer.k_norm.weight"], t[a + ".indexer.k_norm.bias"] = c(lw.idx_k_norm_w), c(lw.idx_k_norm_b)
        kvb = torch.cat([lw.w_kn, lw.w_v.transpose(1, 2)], dim=1).reshape(h * (Dn + Dv), R)
        t[a + ".kv_b_proj.weight"] = c(kvb)
        _put_linear(t, a + ".o_proj", lw.o_proj if lw.o_proj.is_nvfp4 else LinearWeight(c(lw.o_proj.weight)))
        if lw.experts is not None:
            t[m + ".gate.weight"] = c(lw.router_w)
            t[m + ".gate.e_score_correction_bias"] = lw.router_bias.cpu().float()
            _put_experts(t, m + ".experts", lw.experts if lw.experts.is_nvfp4 else lw.experts.to("cpu", dtype), True)
            if lw.shared is not None:
                _put_experts(t, m + ".shared_experts", lw.shared if lw.shared.is_nvfp4 else lw.shared.to("cpu", dtype), False)
        else:
            I = lw.mlp_w13.out_features // 2
            w13 = lw.mlp_w13 if lw.mlp_w13.is_nvfp4 else LinearWeight(c(lw.mlp_w13.weight))
            _put_linear(t, m + ".gate_proj", w13.rows(0, I))
            _put_linear(t, m + ".up_proj", w13.rows(I, 2 * I))
            _put_linear(t, m + ".down_proj", lw.mlp_w2 if lw.mlp_w2.is_nvfp4 else LinearWeight(c(lw.mlp_w2.weight)))
        if lw.eh_proj is not None:
            t[p + ".eh_proj.weight"] = c(lw.eh_proj.weight)
            t[p + ".enorm.weight"], t[p + ".hnorm.weight"] = c(lw.enorm), c(lw.hnorm)
            t[p + ".shared_head.norm.weight"] = c(lw.shared_head_norm)
    fn = "model-00001-of-00001.safetensors"
    save_file({k: v.contiguous() for k, v in t.items()}, os.path.join(out_dir, fn), {"format": "pt"})
    with open(os.path.join(out_dir, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {}, "weight_map": {k: fn for k in t}}, f)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(cfg.to_hf_dict(), f)
    return out_dir
