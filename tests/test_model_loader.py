"""Persistent loader: arena packing, export / import through shared memory between processes, executor
supervision and the control endpoints (reference: `src/run_model_loader.ts`, IPC child fixtures
`tests/fixtures/cuda_ipc_child.ts`)."""
import json
import sys
import time
import urllib.request

import torch

from slopllm_b200.cli import model_loader as ML

from mp_util import _free_port

CHILD = r"""
import json, os, sys, torch
sys.path.insert(0, os.getcwd())
from slopllm_b200.cli.model_loader import attach_from_env
t = attach_from_env(0)
print("CHECKSUM", float(t["a"].double().sum() + t["b"].double().sum()), list(t["b"].shape), str(t["b"].dtype), flush=True)
import time; time.sleep(float(os.environ.get("CHILD_SLEEP", "0")))
"""


def _get(port, path):
    with urllib.request.urlopen(f"http://127.0.0.1:{port}{path}", timeout=10) as r:
        return r.read().decode()


def _post(port, path, obj=None):
    req = urllib.request.Request(f"http://127.0.0.1:{port}{path}", data=json.dumps(obj or {}).encode(), method="POST",
                                 headers={"Content-Type": "application/json"})
    with urllib.request.urlopen(req, timeout=30) as r:
        return json.loads(r.read())


def test_pack_and_views_roundtrip():
    t = {"a": torch.arange(10, dtype=torch.float32), "b": torch.randn(3, 5).to(torch.bfloat16), "c": torch.tensor([1, 2, 3], dtype=torch.uint8)}
    buf, layout = ML.pack_arena(t, "cpu")
    assert all(e["offset"] % 256 == 0 for e in layout)
    v = ML.views_from_arena(buf, layout)
    assert all(torch.equal(v[k], t[k]) for k in t)


def test_loader_keeps_weights_across_executor_restarts(tmp_path):
    t = {"a": torch.arange(1000, dtype=torch.float32), "b": torch.ones(4, 8, dtype=torch.bfloat16)}
    keep = []
    buf, layout = ML.pack_arena(t, "cpu")
    env = {"SLOPLLM_B200_ARENA_IPC_HANDLE_0": ML.export_arena(buf, keep), "SLOPLLM_B200_ARENA_LAYOUT_0": json.dumps(layout),
           "CHILD_SLEEP": "0"}
    ex = ML.Executor(env)
    port = _free_port()
    srv = ML.make_control_server(ex, {"model": "x"}, port)
    import threading
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    try:
        assert json.loads(_get(port, "/status"))["running"] is False
        assert json.loads(_get(port, "/model-args")) == {"model": "x"}
        want = float(t["a"].double().sum() + t["b"].double().sum())
        for attempt in range(2):                                   # spawn, then restart: the arena is mapped again, not rebuilt
            st = _post(port, "/spawn", {"cmd": [sys.executable, "-c", CHILD]}) if attempt == 0 else _post(port, "/restart")
            assert st["cmd"][0] == sys.executable
            t0 = time.time()
            while json.loads(_get(port, "/status"))["running"] and time.time() - t0 < 60:
                time.sleep(0.1)
            out = _get(port, "/follow?live=0")
            assert out.count(f"CHECKSUM {want}") == attempt + 1 and "[4, 8] torch.bfloat16" in out
        assert json.loads(_get(port, "/status"))["restarts"] == 1
        ex.env["CHILD_SLEEP"] = "30"
        _post(port, "/spawn", {"cmd": [sys.executable, "-c", CHILD]})
        time.sleep(1.0)
        assert json.loads(_get(port, "/status"))["running"] is True
        assert _post(port, "/stop")["running"] is False
        # /fork runs a module of this interpreter as the executor
        st = _post(port, "/fork", {"module": "platform"})
        assert st["cmd"][:3] == [sys.executable, "-m", "platform"]
        t0 = time.time()
        while json.loads(_get(port, "/status"))["running"] and time.time() - t0 < 30:
            time.sleep(0.1)
        assert "Linux" in _get(port, "/follow?live=0")
    finally:
        ex.stop()
        srv.shutdown()
        for s in keep:
            s.close()
            try:
                s.unlink()
            except FileNotFoundError:
                pass
