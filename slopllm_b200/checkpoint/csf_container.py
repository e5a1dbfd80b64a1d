"""`lil-nvfp4-csf-checkpoint/1` container: reader with fail-closed contract checks, integrity
verification, source-shard reconstruction, and a builder.

Layout (parity: `src/csf_checkpoint.ts:1-769`, fixture `tests/csf_fixture.ts`):
  manifest.json          identity (schema / codec / family / metadata_sha256), shard records with
                         source/target sizes and sha256, compressed_scale_count
  build-contract.json    same identity + source_names (logical tensor name -> shard file)
  metadata/              config.json, tokenizer files, model.safetensors.index.json ... (hashed)
  receipts/<shard>.json  per shard: sizes, hashes, source_header_base64 (the original safetensors
                         header) and one record per replaced scale tensor
  tensors/<shard>        safetensors: native tensors byte-identical to the source; every replaced
                         `*.weight_scale` becomes `<name>.nvfp4_csf_fixed` (U8) +
                         `<name>.nvfp4_csf_exceptions` (U32)
"""
from __future__ import annotations

import base64
import hashlib
import json
import os
import struct
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

from . import csf_codec as codec
from .csf_codec import CsfContractError
from .safetensors_io import SafetensorsFile, serialize


def _sha(data) -> str:
    return hashlib.sha256(bytes(data)).hexdigest()


def _sha_file(path: str) -> Tuple[str, int]:
    h = hashlib.sha256()
    n = 0
    with open(path, "rb") as f:
        while True:
            b = f.read(1 << 22)
            if not b:
                break
            h.update(b)
            n += len(b)
    return h.hexdigest(), n


def looks_like_csf(root: str) -> bool:
    if any(os.path.exists(os.path.join(root, m)) for m in ("build-contract.json", "receipts")):
        return True
    man = os.path.join(root, "manifest.json")
    if os.path.exists(man):
        with open(man) as f:
            return "-csf-checkpoint/" in f.read()
    return False


def _json(root: str, rel: str):
    p = os.path.join(root, rel)
    try:
        with open(p) as f:
            text = f.read()
    except OSError as e:
        raise CsfContractError(f"CSF container is missing {rel}: {e}")
    try:
        return json.loads(text)
    except json.JSONDecodeError as e:
        raise CsfContractError(f"CSF container {rel} is not valid JSON: {e}")


def _rec(v, what) -> dict:
    if not isinstance(v, dict):
        raise CsfContractError(f"CSF {what} must be a JSON object")
    return v


def _num(v, what) -> int:
    if not isinstance(v, int) or isinstance(v, bool) or v < 0:
        raise CsfContractError(f"CSF {what} must be a non-negative integer")
    return v


def _str(v, what) -> str:
    if not isinstance(v, str) or not v:
        raise CsfContractError(f"CSF {what} must be a non-empty string")
    return v


def _local_name(file: str) -> None:
    if os.path.basename(file) != file or not file.endswith(".safetensors"):
        raise CsfContractError("CSF shard names must be checkpoint-local safetensors files")


@dataclass
class ShardRecord:
    file: str
    source_file_bytes: int
    source_sha256: str
    target_file_bytes: int
    target_sha256: str


@dataclass
class ScaleRecord:
    file: str
    dtype: str
    shape: Tuple[int, int]
    source_bytes: int
    source_sha256: str
    fixed_bytes: int
    exception_bytes: int


class CsfContainer:
    """Opened container.  Construction runs every structural contract check (fail-closed)."""

    def __init__(self, root: str):
        self.root = root
        man = _rec(_json(root, "manifest.json"), "manifest")
        con = _rec(_json(root, "build-contract.json"), "build-contract")
        for key, want in (("schema", codec.SCHEMA), ("codec", codec.CODEC)):
            if man.get(key) != want or con.get(key) != want:
                raise CsfContractError(f"CSF requires {key}={want} in both manifest and build-contract")
        fam = _str(con.get("family"), "family")
        if fam not in codec.SUPPORTED_FAMILIES:
            raise CsfContractError(f"CSF family {fam} is not supported (want one of {', '.join(codec.SUPPORTED_FAMILIES)})")
        if man.get("family") != fam:
            raise CsfContractError("CSF manifest and build-contract must name the same model family")
        self.family = fam
        mm, cm = _rec(man.get("metadata_sha256"), "manifest metadata_sha256"), _rec(con.get("metadata_sha256"), "build-contract metadata_sha256")
        if json.dumps(mm, sort_keys=True) != json.dumps(cm, sort_keys=True):
            raise CsfContractError("CSF manifest and build-contract disagree on metadata hashes")
        self.metadata_sha256: Dict[str, str] = dict(mm)
        self.source_names: Dict[str, str] = {k: _str(v, f"source_names[{k}]") for k, v in _rec(con.get("source_names"), "source_names").items()}
        shards = man.get("shards")
        if not isinstance(shards, list):
            raise CsfContractError("CSF manifest shards must be a list")
        self.shards: Dict[str, ShardRecord] = {}
        for entry in shards:
            it = _rec(entry, "manifest shard")
            file = _str(it.get("file"), "manifest shard file")
            _local_name(file)
            if file in self.shards:
                raise CsfContractError(f"CSF manifest lists shard {file} twice")
            self.shards[file] = ShardRecord(file, _num(it.get("source_file_bytes"), f"shard {file} source_file_bytes"),
                                            _str(it.get("source_sha256"), f"shard {file} source_sha256"),
                                            _num(it.get("target_file_bytes"), f"shard {file} target_file_bytes"),
                                            _str(it.get("target_sha256"), f"shard {file} target_sha256"))
        if set(self.shards) != set(self.source_names.values()):
            raise CsfContractError("CSF manifest and source tensor inventory disagree on shard files")
        self.compressed_scale_count = _num(man.get("compressed_scale_count"), "compressed_scale_count")
        self.scales: Dict[str, ScaleRecord] = {}
        self.receipts: Dict[str, dict] = {}
        for file in self.shards:
            rc = _rec(_json(root, f"receipts/{file}.json"), f"receipt for {file}")
            self.receipts[file] = rc
            for name, item in _rec(rc.get("scales", {}), f"receipt {file} scales").items():
                it = _rec(item, f"scale {name}")
                shape = it.get("shape")
                if it.get("dtype") != "F8_E4M3" or not (isinstance(shape, list) and len(shape) == 2):
                    raise CsfContractError(f"CSF receipt {file} scale {name} has a malformed shape/dtype")
                if name in self.scales:
                    raise CsfContractError(f"CSF scale {name} appears in two receipts")
                self.scales[name] = ScaleRecord(file, it["dtype"], (int(shape[0]), int(shape[1])),
                                                _num(it.get("source_bytes"), f"scale {name} source_bytes"),
                                                _str(it.get("source_sha256"), f"scale {name} source_sha256"),
                                                _num(it.get("fixed_bytes"), f"scale {name} fixed_bytes"),
                                                _num(it.get("exception_bytes"), f"scale {name} exception_bytes"))
        if self.compressed_scale_count != len(self.scales):
            raise CsfContractError(f"CSF manifest compressed_scale_count {self.compressed_scale_count} disagrees with "
                                   f"{len(self.scales)} receipt scale entries")
        # open shards, reconcile physical tensors with the logical inventory
        self.files: Dict[str, SafetensorsFile] = {}
        for file, rec in self.shards.items():
            path = os.path.join(root, "tensors", file)
            if not os.path.exists(path):
                raise CsfContractError(f"CSF container is missing tensors/{file}")
            size = os.path.getsize(path)
            if size != rec.target_file_bytes:
                raise CsfContractError(f"CSF shard {file} extent is {size} bytes, manifest expects {rec.target_file_bytes}")
            st = SafetensorsFile(path)
            self.files[file] = st
            for name in st.names():
                for suf in (codec.FIXED_SUFFIX, codec.EXC_SUFFIX):
                    if name.endswith(suf) and name[: -len(suf)] not in self.scales:
                        raise CsfContractError(f"CSF shard {file} carries planes for unknown scale {name[:-len(suf)]}")
        for name, file in self.source_names.items():
            st = self.files[file]
            if name in self.scales:
                fx, ex = name + codec.FIXED_SUFFIX, name + codec.EXC_SUFFIX
                if fx not in st.tensors or ex not in st.tensors:
                    raise CsfContractError(f"CSF scale {name} is missing a physical plane in {file}")
                rec = self.scales[name]
                if st.meta(fx).nbytes != rec.fixed_bytes or st.meta(ex).nbytes != rec.exception_bytes:
                    raise CsfContractError(f"CSF scale {name} plane sizes disagree with its receipt")
                if st.meta(fx).nbytes != codec.fixed_stream_length(*rec.shape) or rec.source_bytes != rec.shape[0] * rec.shape[1]:
                    raise CsfContractError(f"CSF scale {name} geometry disagrees with its planes")
                wname = name[: -len("_scale")]
                if wname in st.tensors and codec.scale_geometry(st.meta(wname).shape) != rec.shape:
                    raise CsfContractError(f"CSF scale {name} does not match the geometry of {wname}")
            elif name not in st.tensors:
                raise CsfContractError(f"CSF logical tensor {name} is missing from {file}")

    # ---- logical view -------------------------------------------------------------------------------
    def names(self) -> List[str]:
        return list(self.source_names)

    def is_compressed(self, name: str) -> bool:
        return name in self.scales

    def meta(self, name: str):
        """(dtype, shape) of the logical tensor."""
        if name in self.scales:
            return "F8_E4M3", self.scales[name].shape
        m = self.files[self.source_names[name]].meta(name)
        return m.dtype, m.shape

    def planes(self, name: str) -> Tuple[np.ndarray, np.ndarray]:
        st = self.files[self.scales[name].file]
        fixed = np.frombuffer(st.read_bytes(name + codec.FIXED_SUFFIX), dtype=np.uint8)
        exc = np.frombuffer(st.read_bytes(name + codec.EXC_SUFFIX), dtype="<u4")
        return fixed, exc

    def tensor(self, name: str) -> torch.Tensor:
        """Logical tensor (replaced scales are decoded on the CPU)."""
        if name in self.scales:
            rows, cols = self.scales[name].shape
            fixed, exc = self.planes(name)
            return torch.from_numpy(codec.expand_scale_planes(fixed, exc, rows, cols).copy()).view(torch.float8_e4m3fn)
        return self.files[self.source_names[name]].tensor(name)

    def metadata_path(self, rel: str) -> str:
        return os.path.join(self.root, "metadata", rel)

    # ---- integrity --------------------------------------------------------------------------------------
    def verify(self, deep: bool = True) -> List[str]:
        """Recompute hashes and reconcile manifest / receipts / metadata.  Returns the problems."""
        problems: List[str] = []
        for name, want in self.metadata_sha256.items():
            p = self.metadata_path(name)
            if not os.path.exists(p):
                problems.append(f"metadata file {name} is missing")
                continue
            got, _ = _sha_file(p)
            if got != want:
                problems.append(f"metadata file {name} hash {got} does not match recorded {want}")
        for file, rec in self.shards.items():
            rc = self.receipts[file]
            for key, want in (("source_sha256", rec.source_sha256), ("source_file_bytes", rec.source_file_bytes),
                              ("target_sha256", rec.target_sha256), ("target_file_bytes", rec.target_file_bytes)):
                if rc.get(key) != want:
                    problems.append(f"receipt {file} {key} disagrees with the manifest")
            if deep:
                got, n = _sha_file(os.path.join(self.root, "tensors", file))
                if got != rec.target_sha256 or n != rec.target_file_bytes:
                    problems.append(f"shard {file} target hash/size does not match the manifest")
        if deep:
            for name, rec in self.scales.items():
                try:
                    fixed, exc = self.planes(name)
                    logical = codec.expand_scale_planes(fixed, exc, *rec.shape)
                    if _sha(logical.tobytes()) != rec.source_sha256:
                        problems.append(f"scale {name} does not decode to its recorded source bytes")
                except CsfContractError as e:
                    problems.append(f"scale {name}: {e}")
        return problems

    def reconstruct_source_shard(self, file: str) -> bytes:
        """Rebuild the original safetensors shard byte-for-byte from the container."""
        rc = self.receipts[file]
        header = base64.b64decode(_str(rc.get("source_header_base64"), f"receipt {file} source_header_base64"))
        (n,) = struct.unpack("<Q", header[:8])
        meta = json.loads(header[8:8 + n])
        meta.pop("__metadata__", None)
        out = bytearray(header)
        for name, t in sorted(meta.items(), key=lambda kv: kv[1]["data_offsets"][0]):
            if name in self.scales:
                fixed, exc = self.planes(name)
                data = codec.expand_scale_planes(fixed, exc, *self.scales[name].shape).tobytes()
            else:
                data = bytes(self.files[file].read_bytes(name))
            b, e = t["data_offsets"]
            if len(data) != e - b:
                raise CsfContractError(f"CSF tensor {name} reconstructs to {len(data)} bytes, source header expects {e - b}")
            out += data
        rec = self.shards[file]
        if len(out) != rec.source_file_bytes or _sha(out) != rec.source_sha256:
            raise CsfContractError(f"CSF shard {file} does not reconstruct to its recorded source")
        return bytes(out)

    def close(self) -> None:
        for st in self.files.values():
            st.close()


def build_csf_container(source_dir: str, out_dir: str, family: str = "glm53_744b_nvfp4", model_id: str = "local/model",
                        revision: str = "0" * 40) -> Dict[str, int]:
    """Convert a plain NVFP4 safetensors checkpoint directory into a CSF container: every
    `*.weight_scale` (F8_E4M3, 16-row slabs, even columns) is replaced by its two planes."""
    for d in ("metadata", "receipts", "tensors"):
        os.makedirs(os.path.join(out_dir, d), exist_ok=True)
    shard_files = sorted(f for f in os.listdir(source_dir) if f.endswith(".safetensors"))
    weight_map: Dict[str, str] = {}
    shard_records, n_scales, comp_bytes, orig_bytes = [], 0, 0, 0
    for file in shard_files:
        src_path = os.path.join(source_dir, file)
        st = SafetensorsFile(src_path)
        with open(src_path, "rb") as f:
            src_bytes = f.read()
        target: Dict[str, torch.Tensor] = {}
        scale_records = {}
        for name in st.names():
            weight_map[name] = file
            m = st.meta(name)
            ok = (name.endswith(".weight_scale") and m.dtype == "F8_E4M3" and len(m.shape) == 2 and m.shape[0] % 16 == 0
                  and m.shape[1] % 2 == 0)
            if ok:
                logical = np.frombuffer(st.read_bytes(name), dtype=np.uint8).reshape(m.shape)
                try:
                    fixed, exc = codec.compress_scales(logical)
                except CsfContractError:
                    ok = False
            if not ok:
                target[name] = st.tensor(name)
                continue
            target[name + codec.FIXED_SUFFIX] = torch.from_numpy(fixed.copy())
            target[name + codec.EXC_SUFFIX] = torch.from_numpy(exc.astype(np.uint32).view(np.int32).copy()).view(torch.uint32)
            scale_records[name] = {"dtype": "F8_E4M3", "shape": list(m.shape), "source_bytes": int(logical.size),
                                   "source_sha256": _sha(logical.tobytes()), "fixed_bytes": int(fixed.size),
                                   "exception_bytes": int(exc.size * 4)}
            n_scales += 1
            comp_bytes += int(fixed.size + exc.size * 4)
            orig_bytes += int(logical.size)
        data = serialize(target)
        with open(os.path.join(out_dir, "tensors", file), "wb") as f:
            f.write(data)
        rec = {"file": file, "source_file_bytes": len(src_bytes), "source_sha256": _sha(src_bytes),
               "target_file_bytes": len(data), "target_sha256": _sha(data)}
        shard_records.append(rec)
        with open(os.path.join(out_dir, "receipts", f"{file}.json"), "w") as f:
            json.dump({**rec, "source_header_base64": base64.b64encode(src_bytes[:st.data_offset]).decode(),
                       "scales": scale_records, "source_content_address_verified": True}, f)
        st.close()
    meta_sha = {}
    index = json.dumps({"weight_map": weight_map})
    with open(os.path.join(out_dir, "metadata", "model.safetensors.index.json"), "w") as f:
        f.write(index)
    for name in os.listdir(source_dir):
        p = os.path.join(source_dir, name)
        if os.path.isfile(p) and not name.endswith(".safetensors") and name != "model.safetensors.index.json":
            with open(p, "rb") as f:
                data = f.read()
            with open(os.path.join(out_dir, "metadata", name), "wb") as f:
                f.write(data)
    for name in os.listdir(os.path.join(out_dir, "metadata")):
        meta_sha[name] = _sha_file(os.path.join(out_dir, "metadata", name))[0]
    identity = {"schema": codec.SCHEMA, "codec": codec.CODEC, "family": family, "metadata_sha256": meta_sha}
    common = {"compressed_scale_count": n_scales, "source": source_dir, "source_model_id": model_id,
              "source_revision": revision, "source_index_sha256": _sha(index.encode()),
              "source_index_size_semantics": "safetensors_files"}
    with open(os.path.join(out_dir, "manifest.json"), "w") as f:
        json.dump({**identity, **common, "compressed_scale_bytes": comp_bytes, "original_scale_bytes": orig_bytes,
                   "shards": shard_records, "status": "built"}, f)
    with open(os.path.join(out_dir, "build-contract.json"), "w") as f:
        json.dump({**identity, **common, "source_names": weight_map}, f)
    return {"scales": n_scales, "compressed_bytes": comp_bytes, "original_bytes": orig_bytes}


_ = Optional
