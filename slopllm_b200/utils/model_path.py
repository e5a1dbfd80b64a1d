"""Locate checkpoints: a directory as given, or a Hugging Face hub id resolved inside the local
cache (`$HF_HOME/hub/models--org--name/snapshots/<refs/main>`); list a snapshot's safetensors
shards.  Reference: `src/model_path.ts:1-59`."""
from __future__ import annotations

import json
import os
from typing import List


class ModelNotFoundError(FileNotFoundError):
    pass


def resolve_model_path(repo_id_or_dir: str) -> str:
    if os.path.isdir(repo_id_or_dir):
        return repo_id_or_dir
    hf_home = os.environ.get("HF_HOME") or os.path.join(os.path.expanduser("~"), ".cache", "huggingface")
    model_dir = os.path.join(hf_home, "hub", "models--" + repo_id_or_dir.replace("/", "--"))
    if not os.path.isdir(model_dir):
        raise ModelNotFoundError(f'model "{repo_id_or_dir}" not found in the Hugging Face cache\n  looked at: {model_dir}\n'
                                 f"  HF_HOME: {hf_home}\n  download with: huggingface-cli download {repo_id_or_dir}")
    ref = os.path.join(model_dir, "refs", "main")
    if not os.path.isfile(ref):
        raise ModelNotFoundError(f'no refs/main for "{repo_id_or_dir}": the model may not be fully downloaded\n  expected: {ref}')
    with open(ref) as f:
        commit = f.read().strip()
    snap = os.path.join(model_dir, "snapshots", commit)
    if not os.path.isdir(snap):
        raise ModelNotFoundError(f'snapshot directory not found for "{repo_id_or_dir}"\n  expected: {snap}\n  commit: {commit}')
    return snap


def list_safetensors_shards(snapshot_dir: str) -> List[str]:
    index = os.path.join(snapshot_dir, "model.safetensors.index.json")
    if not os.path.isfile(index):
        files = sorted(f for f in os.listdir(snapshot_dir) if f.endswith(".safetensors"))
        if not files:
            raise FileNotFoundError(f"no safetensors files found in {snapshot_dir}")
        return [os.path.join(snapshot_dir, f) for f in files]
    with open(index) as f:
        weight_map = json.load(f)["weight_map"]
    seen, out = set(), []
    for fn in weight_map.values():
        if fn not in seen:
            seen.add(fn)
            out.append(os.path.join(snapshot_dir, fn))
    return out
