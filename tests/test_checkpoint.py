"""safetensors IO, CSF codec and container (mirrors `tests/test_csf_codec.ts`,
`tests/test_csf_checkpoint.ts`: build a valid container, then corrupt it field by field)."""
import json
import os

import numpy as np
import pytest
import torch

from slopllm_b200.checkpoint import csf_codec as codec
from slopllm_b200.checkpoint.csf_codec import CsfContractError
from slopllm_b200.checkpoint.csf_container import CsfContainer, build_csf_container
from slopllm_b200.checkpoint.safetensors_io import SafetensorsFile, save_file
from slopllm_b200.checkpoint.source import open_checkpoint_source
from slopllm_b200.checkpoint.weight_type import resolve_weight_type
from slopllm_b200.ops import quant


def _scales(rows, cols, seed=0, spread=True):
    rng = np.random.default_rng(seed)
    base = rng.integers(0x20, 0x50, size=(rows, 1))
    s = base + rng.integers(0, 16, size=(rows, cols))
    if spread:                                   # a few values outside the 4-bit window -> exceptions
        idx = rng.integers(0, rows * cols, size=20)
        s.reshape(-1)[idx] = rng.integers(0x60, 0x7F, size=20)
    return np.clip(s, 0, 0x7E).astype(np.uint8)


def test_safetensors_roundtrip(tmp_path):
    t = {"a": torch.arange(12, dtype=torch.float32).reshape(3, 4), "b": torch.tensor([1, 2, 3], dtype=torch.uint8),
         "c": torch.randn(4, 8).to(torch.bfloat16), "s": torch.tensor(2.5), "e": torch.rand(2, 16).to(torch.float8_e4m3fn)}
    p = str(tmp_path / "x.safetensors")
    save_file(t, p, {"format": "pt"})
    st = SafetensorsFile(p)
    assert st.metadata == {"format": "pt"} and set(st.names()) == set(t)
    for k, v in t.items():
        got = st.tensor(k)
        assert got.dtype == v.dtype and got.shape == v.shape
        assert torch.equal(got.reshape(-1).view(torch.uint8), v.contiguous().reshape(-1).view(torch.uint8))
    with open(p, "r+b") as f:
        f.write(b"\xff" * 8)
    with pytest.raises(ValueError):
        SafetensorsFile(p)


def test_weight_type_resolution():
    kinds = {"x.weight_scale": "F8_E4M3", "y.weight_scale": "U8", "z.weight_scale_inv": "F32"}
    look = kinds.get
    assert resolve_weight_type("x.weight", "U8", look) == "U8_NVFP4"
    assert resolve_weight_type("y.weight", "U8", look) == "U8_MXFP4"
    assert resolve_weight_type("z.weight", "F8_E4M3", look) == "F8_E4M3_BLOCK"
    assert resolve_weight_type("w.weight", "BF16", look) == "BF16"
    assert resolve_weight_type("q.weight", "U8", look) == "U8"


def test_codec_roundtrip_window_slice_concat():
    s = _scales(64, 24, 1)
    fixed, exc = codec.compress_scales(s)
    assert fixed.size == codec.fixed_stream_length(64, 24) and exc.size > 0
    assert np.array_equal(codec.expand_scale_planes(fixed, exc, 64, 24), s)
    assert np.array_equal(codec.expand_scale_window(fixed, exc, 64, 24, 17, 30, 3, 11), s[17:47, 3:14])
    f2, e2 = codec.slice_scale_planes(fixed, exc, 64, 24, (16, 48), (4, 20))
    assert np.array_equal(codec.expand_scale_planes(f2, e2, 32, 16), s[16:48, 4:20])
    f3, e3 = codec.slice_scale_planes(fixed, exc, 64, 24, (48, 64), (0, 24), out_rows=32, out_columns=28)
    padded = codec.expand_scale_planes(f3, e3, 32, 28)
    assert np.array_equal(padded[:16, :24], s[48:64]) and np.all(padded[16:] == codec.PADDED_SCALE_CODE)
    assert np.array_equal(padded[:16, 24:], np.repeat(f3.reshape(2, -1)[0, :16, None], 4, axis=1))
    other = _scales(64, 24, 2)
    fo, eo = codec.compress_scales(other)
    ff, ef = codec.concat_fc1_scale_planes((fixed, exc), (fo, eo), 64, 24)
    assert np.array_equal(codec.expand_scale_planes(ff, ef, 128, 24), np.concatenate([s, other]))
    assert codec.tp_extent(2048, 3, 8, 16) == (768, 1024)


def test_codec_contract_violations():
    s = _scales(32, 8, 3)
    fixed, exc = codec.compress_scales(s)
    with pytest.raises(CsfContractError):
        codec.expand_scale_planes(fixed[:-1], exc, 32, 8)
    bad = fixed.copy()
    bad[0] = 250
    with pytest.raises(CsfContractError):
        codec.expand_scale_planes(bad, exc, 32, 8)
    with pytest.raises(CsfContractError):
        codec.expand_scale_planes(fixed, exc[::-1].copy(), 32, 8)                  # unsorted
    with pytest.raises(CsfContractError):
        codec.expand_scale_planes(fixed, np.array([(0x7F << 24) | 5], dtype="<u4"), 32, 8)   # NaN code
    with pytest.raises(CsfContractError):
        codec.expand_scale_planes(fixed, np.array([32 * 8], dtype="<u4"), 32, 8)   # out of range
    with pytest.raises(CsfContractError):
        codec.fixed_stream_length(30, 8)
    with pytest.raises(CsfContractError):
        codec.slice_scale_planes(fixed, exc, 32, 8, (8, 24), (0, 8))
    with pytest.raises(CsfContractError):
        codec.tp_extent(100, 0, 8, 16)


def _plain_checkpoint(d):
    g = torch.Generator().manual_seed(0)
    tensors = {}
    for proj, (n, k) in {"gate_proj": (32, 64), "up_proj": (32, 64), "down_proj": (64, 32)}.items():
        w, s, g2 = quant.random_nvfp4((n, k), g)
        pfx = f"model.layers.3.mlp.experts.0.{proj}"
        tensors[pfx + ".weight"] = w
        tensors[pfx + ".weight_scale"] = s
        tensors[pfx + ".weight_scale_2"] = g2
        tensors[pfx + ".input_scale"] = torch.tensor(1.0)
    tensors["model.norm.weight"] = torch.full((8,), 1.5)
    os.makedirs(d, exist_ok=True)
    save_file(tensors, os.path.join(d, "model-00001-of-00001.safetensors"))
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump({"model_type": "glm_moe_dsa", "hidden_size": 64}, f)
    return tensors


def test_container_build_open_verify_reconstruct(tmp_path):
    src, out = str(tmp_path / "src"), str(tmp_path / "csf")
    tensors = _plain_checkpoint(src)
    stats = build_csf_container(src, out)
    assert stats["scales"] == 3
    c = CsfContainer(out)
    assert c.verify() == []
    source = open_checkpoint_source(out)
    assert source.csf is not None and set(source.names()) == set(tensors)
    for k, v in tensors.items():
        assert torch.equal(source.tensor(k).reshape(-1).view(torch.uint8), v.contiguous().reshape(-1).view(torch.uint8)), k
    planes = source.csf_planes("model.layers.3.mlp.experts.0.down_proj.weight_scale")
    assert planes is not None and planes[2] == (64, 2)
    with open(os.path.join(src, "model-00001-of-00001.safetensors"), "rb") as f:
        assert c.reconstruct_source_shard("model-00001-of-00001.safetensors") == f.read()
    plain = open_checkpoint_source(src)
    assert plain.csf is None and set(plain.names()) == set(tensors)


def _mutate(root, rel, fn):
    p = os.path.join(root, rel)
    with open(p) as f:
        d = json.load(f)
    fn(d)
    with open(p, "w") as f:
        json.dump(d, f)


@pytest.mark.parametrize("case", ["schema", "family", "count", "dup_shard", "missing_receipt", "meta_hash", "shard_size",
                                  "plane_size", "target_hash"])
def test_container_rejects_corruption(tmp_path, case):
    src, out = str(tmp_path / "src"), str(tmp_path / "csf")
    _plain_checkpoint(src)
    build_csf_container(src, out)
    shard = "model-00001-of-00001.safetensors"
    if case == "schema":
        _mutate(out, "manifest.json", lambda d: d.__setitem__("schema", "lil-nvfp4-csf-checkpoint/2"))
    elif case == "family":
        _mutate(out, "build-contract.json", lambda d: d.__setitem__("family", "other"))
    elif case == "count":
        _mutate(out, "manifest.json", lambda d: d.__setitem__("compressed_scale_count", 7))
    elif case == "dup_shard":
        _mutate(out, "manifest.json", lambda d: d["shards"].append(dict(d["shards"][0])))
    elif case == "missing_receipt":
        os.remove(os.path.join(out, "receipts", shard + ".json"))
    elif case == "meta_hash":
        _mutate(out, "manifest.json", lambda d: d["metadata_sha256"].__setitem__("config.json", "0" * 64))
    elif case == "shard_size":
        with open(os.path.join(out, "tensors", shard), "ab") as f:
            f.write(b"\0")
    elif case == "plane_size":
        _mutate(out, f"receipts/{shard}.json", lambda d: next(iter(d["scales"].values())).__setitem__("fixed_bytes", 1))
    if case == "target_hash":
        p = os.path.join(out, "tensors", shard)
        data = bytearray(open(p, "rb").read())
        data[-1] ^= 0xFF
        open(p, "wb").write(bytes(data))
        assert any("target hash" in m for m in CsfContainer(out).verify())
        return
    with pytest.raises(CsfContractError):
        CsfContainer(out)


def test_model_save_load_roundtrip_tp_and_csf(tmp_path):
    """Random model -> HF-named safetensors -> CSF container -> load (TP=1 and TP=2 shards) gives the
    same tensors as sharding the in-memory model."""
    from slopllm_b200.checkpoint.loader import load_model, save_model
    from slopllm_b200.config import GlmMoeDsaConfig
    from slopllm_b200.models.weights import random_model
    cfg = GlmMoeDsaConfig.tiny()
    cfg.moe_intermediate_size = 128
    full = random_model(cfg, 0, dtype=torch.bfloat16)
    src = save_model(cfg, full, str(tmp_path / "hf"))
    out = str(tmp_path / "csf")
    assert build_csf_container(src, out)["scales"] > 0
    for root in (src, out):
        for W in (1, 2):
            for r in range(W):
                cfg2, got = load_model(root, "cpu", torch.bfloat16, r, W)
                want = random_model(cfg, 0, dtype=torch.bfloat16, tp_rank=r, tp_world=W)
                assert cfg2.hidden_size == cfg.hidden_size and len(got.layers) == len(want.layers)
                assert torch.equal(got.lm_head.weight, want.lm_head.weight)
                for a, b in zip(got.layers, want.layers):
                    for k, v in b.__dict__.items():
                        u = getattr(a, k)
                        if isinstance(v, torch.Tensor):
                            assert torch.equal(u.float(), v.float()), k
                        elif hasattr(v, "weight"):
                            assert torch.equal(u.weight, v.weight), k
                            if v.scale is not None:
                                assert torch.equal(u.scale.view(torch.uint8), v.scale.view(torch.uint8)), k
                        elif hasattr(v, "w13"):
                            assert torch.equal(u.w13, v.w13) and torch.equal(u.w2, v.w2), k
                            if v.s13 is not None:
                                assert torch.equal(u.s13.view(torch.uint8), v.s13.view(torch.uint8)), k
                                assert torch.equal(u.s2.view(torch.uint8), v.s2.view(torch.uint8)), k


@pytest.mark.gpu
def test_csf_gpu_decode_matches_cpu_codec():
    from slopllm_b200.checkpoint.csf_gpu import check_decode_status, decode_csf_scales
    s = _scales(128, 48, 5)
    fixed, exc = codec.compress_scales(s)
    full = decode_csf_scales(fixed, exc, 128, 48, 0, 128, 0, 48, "cuda")
    assert np.array_equal(full.view(torch.uint8).cpu().numpy(), s)
    win = decode_csf_scales(fixed, exc, 128, 48, 32, 64, 8, 24, "cuda")
    assert np.array_equal(win.view(torch.uint8).cpu().numpy(), s[32:96, 8:32])
    check_decode_status("cuda")
    bad = fixed.copy()
    bad[1] = 251
    decode_csf_scales(bad, exc[::-1].copy(), 128, 48, 0, 128, 0, 48, "cuda")
    with pytest.raises(CsfContractError) as ei:
        check_decode_status("cuda")
    assert "row base" in str(ei.value) and "unsorted" in str(ei.value)


def test_native_mmap_windows_match_slices(tmp_path):
    """The C++ runtime's strided window copy against plain slicing of the mapped tensors, and its bounds checks."""
    import pytest
    from slopllm_b200.checkpoint.safetensors_io import SafetensorsFile, save_file
    from slopllm_b200.runtime.native_runtime import MappedFile
    a = torch.randn(300, 200).to(torch.bfloat16)
    b = torch.arange(1000, dtype=torch.int32)
    c = torch.randint(0, 255, (4096, 1024), dtype=torch.uint8)          # 4 MiB: split over the copy threads
    path = str(tmp_path / "x.safetensors")
    save_file({"a": a, "b": b, "c": c, "s": torch.ones(())}, path)
    f = SafetensorsFile(path)
    assert torch.equal(f.window("a"), a) and f.window("a").is_contiguous()
    assert torch.equal(f.window("a", (10, 77), (16, 100)), a[10:77, 16:100])
    assert torch.equal(f.window("a", cols=(100, 200)), a[:, 100:200])
    assert torch.equal(f.window("b", (5, 900)), b[5:900])
    assert torch.equal(f.window("c", (1, 4000), (8, 1000), threads=8), c[1:4000, 8:1000])
    assert f.window("a", (5, 5)).shape == (0, 200)
    assert f.window("s") is None                                         # 0-d: the caller reads tensor()
    with pytest.raises(IndexError):
        f.window("a", (0, 301))
    f.close()
    m = MappedFile(path)
    buf = torch.empty(64, dtype=torch.uint8)
    with pytest.raises(ValueError):
        m.copy_rows(m.size - 32, 64, 64, 1, buf.data_ptr())              # runs past the end of the file
    with pytest.raises(ValueError):
        m.copy_rows(0, 8, 16, 4, buf.data_ptr())                         # rows would overlap
    m.copy_rows(m.size - 64, 64, 64, 1, buf.data_ptr())
    m.advise(0, m.size)
    m.close()
    with pytest.raises(OSError):
        MappedFile(str(tmp_path / "missing.safetensors"))
