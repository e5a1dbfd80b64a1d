"""The serving stack end to end on a GPU: `python -m slopllm_b200 serve` with random weights of a small
glm_moe_dsa model, CUDA kernels, CUDA-graph decode, on-device sampling, MTP drafts; one plain and one streamed
chat completion plus the metrics page."""
import json
import subprocess
import sys
import time
import urllib.request

import pytest

from mp_util import _free_port

pytestmark = pytest.mark.gpu


def _wait_up(proc, port, seconds=240):
    for _ in range(seconds * 2):
        try:
            with urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=2) as r:
                return r.status == 200
        except Exception:  # noqa: BLE001
            if proc.poll() is not None:
                return False
            time.sleep(0.5)
    return False


@pytest.mark.parametrize("mtp", [0, 2])
def test_serve_on_gpu(mtp):
    port = _free_port()
    cmd = [sys.executable, "-m", "slopllm_b200", "serve", "--random-init", "tiny", "--batch-size", "2", "--chunk-size", "64",
           "--max-pages", "64", "--port", str(port), "--max-model-len", "2048"]
    if mtp:
        cmd += ["--mtp", str(mtp)]
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    try:
        assert _wait_up(proc, port), proc.stdout.read() if proc.poll() is not None else "server did not come up"
        body = {"model": "tiny", "messages": [{"role": "user", "content": "hello there"}], "max_tokens": 12, "temperature": 0.7, "top_p": 0.9}
        req = urllib.request.Request(f"http://127.0.0.1:{port}/v1/chat/completions", data=json.dumps(body).encode(),
                                     headers={"Content-Type": "application/json"})
        with urllib.request.urlopen(req, timeout=180) as r:
            out = json.loads(r.read())
        assert 1 <= out["usage"]["completion_tokens"] <= 12
        body.update(stream=True, temperature=0.0, stream_options={"include_usage": True})
        req = urllib.request.Request(f"http://127.0.0.1:{port}/v1/chat/completions", data=json.dumps(body).encode(),
                                     headers={"Content-Type": "application/json"})
        with urllib.request.urlopen(req, timeout=180) as r:
            text = r.read().decode()
        assert "data: [DONE]" in text and '"usage"' in text
        with urllib.request.urlopen(f"http://127.0.0.1:{port}/metrics", timeout=10) as r:
            metrics = r.read().decode()
        assert "vllm:generation_tokens_total" in metrics
        if mtp:
            assert "vllm:spec_decode_num_drafts_total" in metrics
    finally:
        proc.terminate()
        try:
            proc.wait(timeout=30)
        except subprocess.TimeoutExpired:
            proc.kill()
