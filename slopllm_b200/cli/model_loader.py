"""Persistent model loader: a resident parent process loads the weights ONCE into one arena per
rank, exports the arena (CUDA IPC handle on a GPU, POSIX shared memory on the CPU) together with the
allocation layout through environment variables, and runs the executor (server, benchmark, chat)
as a child that maps the arena instead of loading the checkpoint again.  Executors can be stopped,
restarted or replaced by another command while the weights stay resident.

    python -m slopllm_b200.cli.model_loader --random-init tiny --cpu --control-port 8100 -- \\
        python -m slopllm_b200.cli.serve --from-loader --port 8000

Environment handed to the executor (n = rank):
    SLOPLLM_B200_ARENA_IPC_HANDLE_n   hex CUDA IPC handle + offset, or `shm:<name>` on the CPU
    SLOPLLM_B200_ARENA_LAYOUT_n       JSON [{"name", "offset", "shape", "dtype"}, ...]
    SLOPLLM_B200_MODEL_ARGS           JSON of the loader's model arguments (so both sides agree)

Control HTTP (127.0.0.1:--control-port): GET /status, GET /model-args, GET /follow (last 128 KB of the
executor's output, then live), POST /spawn {"cmd": [...]}, POST /stop, POST /restart.

Reference: `src/run_model_loader.ts:1-421` (same handshake with `SLOPLLM_ARENA_IPC_HANDLE_n`,
`SLOPLLM_ARENA_LAYOUT_n`, `SLOPLLM_MODEL_LAYOUT_n`, control endpoints `:302-375`).
"""
from __future__ import annotations

import argparse
import collections
import ctypes as C
import json
import os
import subprocess
import sys
import threading
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Dict, List, Optional

import torch

ENV_PREFIX = "SLOPLLM_B200_"
_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16, "uint8": torch.uint8,
           "int32": torch.int32, "int64": torch.int64, "float8_e4m3fn": torch.float8_e4m3fn}


# ---- arena: pack named tensors into one buffer and describe it --------------------------------------------
def pack_arena(tensors: Dict[str, torch.Tensor], device, alignment: int = 256):
    """Copy the tensors into one contiguous uint8 buffer on `device`; returns (buffer, layout)."""
    layout, off = [], 0
    for name, t in tensors.items():
        off = (off + alignment - 1) // alignment * alignment
        layout.append({"name": name, "offset": off, "shape": list(t.shape), "dtype": str(t.dtype).replace("torch.", "")})
        off += t.numel() * t.element_size()
    buf = torch.empty(max(off, 1), dtype=torch.uint8, device=device)
    for ent, t in zip(layout, tensors.values()):
        n = t.numel() * t.element_size()
        buf[ent["offset"]:ent["offset"] + n].copy_(t.contiguous().view(-1).view(torch.uint8))
    return buf, layout


def views_from_arena(buf: torch.Tensor, layout: List[dict]) -> Dict[str, torch.Tensor]:
    out = {}
    for ent in layout:
        dt = _DTYPES[ent["dtype"]]
        n = 1
        for s in ent["shape"]:
            n *= s
        nbytes = n * torch.empty((), dtype=dt).element_size()
        out[ent["name"]] = buf[ent["offset"]:ent["offset"] + nbytes].view(dt).view(*ent["shape"])
    return out


# ---- export / import -------------------------------------------------------------------------------------------
class _CudaArray:
    """Zero-copy view of a raw device pointer for torch (`__cuda_array_interface__`)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


def export_arena(buf: torch.Tensor, keep: list) -> str:
    if buf.is_cuda:
        from ..ops import native as N
        lib = N.kernels()
        lib.sl_ipc_export.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_ulonglong)]
        handle, offset = (C.c_ubyte * 64)(), C.c_ulonglong(0)
        N.check(lib.sl_ipc_export(buf.data_ptr(), handle, C.byref(offset)), "sl_ipc_export")
        return bytes(handle).hex() + ":" + str(int(offset.value)) + ":" + str(buf.numel())
    from multiprocessing import shared_memory
    shm = shared_memory.SharedMemory(create=True, size=max(1, buf.numel()))
    shm.buf[:buf.numel()] = buf.numpy().tobytes()
    keep.append(shm)
    return f"shm:{shm.name}:{buf.numel()}"


def import_arena(spec: str, device, keep: list) -> torch.Tensor:
    if spec.startswith("shm:"):
        from multiprocessing import shared_memory
        _, name, n = spec.split(":")
        shm = shared_memory.SharedMemory(name=name)
        try:
            # the segment belongs to the loader: an executor that exits must not unlink it
            from multiprocessing import resource_tracker
            resource_tracker.unregister(shm._name, "shared_memory")
        except Exception:  # noqa: BLE001
            pass
        keep.append(shm)
        return torch.frombuffer(shm.buf, dtype=torch.uint8, count=int(n))
    from ..ops import native as N
    hexh, off, n = spec.split(":")
    lib = N.kernels()
    lib.sl_ipc_open.argtypes = [C.c_void_p, C.c_ulonglong, C.POINTER(C.c_void_p)]
    out = C.c_void_p()
    hbuf = (C.c_ubyte * 64).from_buffer_copy(bytes.fromhex(hexh))
    N.check(lib.sl_ipc_open(hbuf, int(off), C.byref(out)), "sl_ipc_open")
    return torch.as_tensor(_CudaArray(int(out.value), int(n)), device=device)


def attach_from_env(rank: int = 0, device="cpu", keep: Optional[list] = None) -> Optional[Dict[str, torch.Tensor]]:
    """Executor side: the loader's tensors, or None when this process was not started by a loader."""
    spec = os.environ.get(f"{ENV_PREFIX}ARENA_IPC_HANDLE_{rank}")
    lay = os.environ.get(f"{ENV_PREFIX}ARENA_LAYOUT_{rank}")
    if not spec or not lay:
        return None
    keep = keep if keep is not None else _KEEP
    return views_from_arena(import_arena(spec, torch.device(device), keep), json.loads(lay))


_KEEP: list = []


# ---- executor supervision + control server -------------------------------------------------------------------
class Executor:
    def __init__(self, env: Dict[str, str]):
        self.env = env
        self.cmd: List[str] = []
        self.proc: Optional[subprocess.Popen] = None
        self.log = collections.deque(maxlen=2048)             # recent output lines (~128 KB)
        self.restarts = 0
        self._lock = threading.Lock()
        self._cond = threading.Condition()

    def spawn(self, cmd: List[str]) -> None:
        with self._lock:
            self.stop()
            self.cmd = list(cmd)
            self.proc = subprocess.Popen(cmd, env={**os.environ, **self.env}, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                                         text=True, bufsize=1)
            threading.Thread(target=self._pump, args=(self.proc,), daemon=True).start()

    def _pump(self, proc) -> None:
        for line in proc.stdout:
            with self._cond:
                self.log.append(line)
                self._cond.notify_all()
        proc.wait()
        with self._cond:
            self.log.append(f"[loader] executor exited with code {proc.returncode}\n")
            self._cond.notify_all()

    def stop(self) -> None:
        if self.proc is not None and self.proc.poll() is None:
            self.proc.terminate()                                # exactly the child this loader started
            try:
                self.proc.wait(timeout=20)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        self.proc = None

    def restart(self) -> None:
        self.restarts += 1
        self.spawn(self.cmd)

    def status(self) -> dict:
        p = self.proc
        return {"running": p is not None and p.poll() is None, "pid": p.pid if p else None,
                "exit_code": p.poll() if p else None, "cmd": self.cmd, "restarts": self.restarts}


def make_control_server(ex: Executor, model_args: dict, port: int, on_quit=None) -> ThreadingHTTPServer:
    class H(BaseHTTPRequestHandler):
        def log_message(self, *a):                                 # noqa: D102
            pass

        def _json(self, code, obj):
            body = json.dumps(obj).encode()
            self.send_response(code)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(body)))
            self.end_headers()
            self.wfile.write(body)

        def do_GET(self):                                          # noqa: N802
            if self.path == "/status":
                self._json(200, ex.status())
            elif self.path == "/model-args":
                self._json(200, model_args)
            elif self.path.startswith("/follow"):
                self.send_response(200)
                self.send_header("Content-Type", "text/plain; charset=utf-8")
                self.end_headers()
                live = "live=0" not in self.path
                sent = 0
                try:
                    while True:
                        with ex._cond:
                            lines = list(ex.log)
                            if sent >= len(lines):
                                if not live or not ex.status()["running"]:
                                    break
                                ex._cond.wait(timeout=1.0)
                                continue
                        self.wfile.write("".join(lines[sent:]).encode())
                        self.wfile.flush()
                        sent = len(lines)
                        if not live:
                            break
                except (BrokenPipeError, ConnectionResetError):
                    pass
            else:
                self._json(404, {"error": "not found"})

        def do_POST(self):                                         # noqa: N802
            n = int(self.headers.get("Content-Length", "0") or 0)
            body = json.loads(self.rfile.read(n) or b"{}") if n else {}
            if self.path == "/spawn":
                cmd = body.get("cmd")
                if not isinstance(cmd, list) or not cmd:
                    return self._json(400, {"error": "cmd must be a non-empty list"})
                ex.spawn([str(c) for c in cmd])
                self._json(200, ex.status())
            elif self.path == "/fork":
                # run one of this interpreter's modules as the executor (the reference forks a script of its own runtime,
                # `src/run_model_loader.ts:302-375`): {"module": "slopllm_b200.cli.serve", "args": ["--port", "8000"]}
                module = body.get("module")
                if not isinstance(module, str) or not module:
                    return self._json(400, {"error": "module must be a dotted module name"})
                ex.spawn([sys.executable, "-m", module, *[str(a) for a in body.get("args") or []]])
                self._json(200, ex.status())
            elif self.path == "/stop":
                ex.stop()
                self._json(200, ex.status())
                if body.get("quit") and on_quit:
                    on_quit()
            elif self.path == "/restart":
                ex.restart()
                self._json(200, ex.status())
            else:
                self._json(404, {"error": "not found"})

    return ThreadingHTTPServer(("127.0.0.1", port), H)


def model_tensors(model) -> Dict[str, torch.Tensor]:
    """Flat name -> tensor map of a model's weights (every tensor reachable from `model.w`)."""
    from ..runtime.workspace import walk_tensors
    out: Dict[str, torch.Tensor] = {}
    walk_tensors(model.w, lambda t: out.setdefault(f"t{len(out):05d}", t))
    return out


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    cmd: List[str] = []
    if "--" in argv:
        i = argv.index("--")
        argv, cmd = argv[:i], argv[i + 1:]
    from .model_cli import add_model_args, build_runtime
    ap = argparse.ArgumentParser(prog="slopllm_b200.cli.model_loader")
    add_model_args(ap)
    ap.add_argument("--control-port", type=int, default=8100)
    args = ap.parse_args(argv)
    rt = build_runtime(args, with_scheduler=False)
    rank = rt.ctx.rank
    keep: list = []
    buf, layout = pack_arena(model_tensors(rt.model), rt.ctx.device)
    env = {f"{ENV_PREFIX}ARENA_IPC_HANDLE_{rank}": export_arena(buf, keep), f"{ENV_PREFIX}ARENA_LAYOUT_{rank}": json.dumps(layout),
           f"{ENV_PREFIX}MODEL_ARGS": json.dumps(vars(args))}
    ex = Executor(env)
    if cmd:
        ex.spawn(cmd)
    done = threading.Event()
    srv = make_control_server(ex, vars(args), args.control_port + rank, on_quit=done.set)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    print(f"[loader] rank {rank}: {len(layout)} tensors, {buf.numel() / 1e9:.2f} GB resident; control on 127.0.0.1:{args.control_port + rank}",
          file=sys.stderr, flush=True)
    try:
        done.wait()
    except KeyboardInterrupt:
        pass
    ex.stop()
    srv.shutdown()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
