"""OpenAI-compatible HTTP server (asyncio, no third-party web framework).

Endpoints and behaviour follow `src/openai-server.ts:963-1030`:
  POST /v1/chat/completions   (stream / non-stream, stream_options.include_usage, tools,
                               reasoning_content, stop strings, max_tokens | max_completion_tokens,
                               temperature / top_p / top_k / repetition_penalty (alias
                               frequency_penalty) / presence_penalty, chat_template_kwargs)
  POST /tokenize
  POST /admin/flush_gpu_cache, POST /admin/flush_host_cache   (admin key)
  GET  /metrics  (Prometheus text, vLLM-compatible metric names), /v1/models, /version, /health
Bearer authentication (`--api-key`, `--admin-api-key`), CORS preflight.

The scheduler runs in its own thread; tokens cross into the event loop with
`loop.call_soon_threadsafe`.
"""
from __future__ import annotations

import asyncio
import json
import time
import uuid
from typing import Dict, List, Optional

from .. import __version__
from ..config import EngineConfig, SamplingParams, env_flag, env_str
from ..scheduler.scheduler import GenerationRequest, GenerationScheduler
from .parsers import ChatModelParser, GlmParser, check_stop_sequences, resolve_control_tokens, starts_in_reasoning

CORS = {"Access-Control-Allow-Origin": "*", "Access-Control-Allow-Headers": "authorization, content-type",
        "Access-Control-Allow-Methods": "GET, POST, OPTIONS"}


class HttpError(Exception):
    def __init__(self, status: int, message: str, etype: str = "invalid_request_error", param: Optional[str] = None,
                 code: Optional[str] = None):
        super().__init__(message)
        self.status, self.message, self.etype, self.param, self.code = status, message, etype, param, code

    def body(self) -> dict:
        err = {"message": self.message, "type": self.etype}
        if self.param:
            err["param"] = self.param
        if self.code:
            err["code"] = self.code
        return {"error": err}


def render_metrics(m, pending: int, kv, batch_size: int, chunk_size: int, max_model_len: int, cp_world: int = 1) -> str:
    """Prometheus exposition text; metric names match `src/openai-server.ts:335-407`."""
    waiting = max(0, pending - max(0, batch_size - m.running_requests))
    used = (kv.num_pages - kv.free_pages) / kv.num_pages if kv.num_pages else 0.0
    lines = [
        "# TYPE vllm:num_requests_running gauge", f"vllm:num_requests_running {m.running_requests}",
        "# TYPE vllm:num_requests_waiting gauge", f"vllm:num_requests_waiting {waiting}",
        "# TYPE vllm:generation_tokens_total counter", f"vllm:generation_tokens_total {m.generation_tokens_total}",
        "# TYPE vllm:prompt_tokens_total counter", f"vllm:prompt_tokens_total {m.prompt_tokens_total}",
        "# TYPE vllm:prefix_cache_hits_total counter", f"vllm:prefix_cache_hits_total {m.cached_prompt_tokens_total}",
        "# TYPE vllm:spec_decode_num_drafts_total counter", f"vllm:spec_decode_num_drafts_total {m.spec_decode_num_drafts_total}",
        "# TYPE vllm:spec_decode_num_draft_tokens_total counter",
        f"vllm:spec_decode_num_draft_tokens_total {m.spec_decode_num_draft_tokens_total}",
        "# TYPE vllm:spec_decode_num_accepted_tokens_total counter",
        f"vllm:spec_decode_num_accepted_tokens_total {m.spec_decode_num_accepted_tokens_total}",
        "# TYPE vllm:request_success_total counter", f"vllm:request_success_total {m.request_success_total}",
        "# TYPE vllm:kv_cache_usage_perc gauge", f"vllm:kv_cache_usage_perc {used}",
        "# TYPE vllm:cache_config_info gauge",
        f'vllm:cache_config_info{{block_size="{kv.tokens_per_page}",num_gpu_blocks="{kv.num_pages}",'
        f'max_total_num_tokens="{kv.num_pages * kv.tokens_per_page}",cp_world_size="{cp_world}"}} 1',
        "# TYPE vllm:scheduler_config_info gauge",
        f'vllm:scheduler_config_info{{max_num_seqs="{batch_size}",max_num_batched_tokens="{chunk_size}",'
        f'max_model_len="{max_model_len}"}} 1',
        "# TYPE vllm:request_prefill_time_seconds histogram",
        f'vllm:request_prefill_time_seconds_bucket{{le="+Inf"}} {m.prefill_time_seconds_count}',
        f"vllm:request_prefill_time_seconds_sum {m.prefill_time_seconds_sum}",
        f"vllm:request_prefill_time_seconds_count {m.prefill_time_seconds_count}",
        "# TYPE glm:phase_seconds_total counter", "# TYPE glm:phase_count_total counter",
        "# TYPE glm:collective_timeouts_total counter", f"glm:collective_timeouts_total {m.collective_timeouts_total}",
        "# TYPE glm:rank_failures_total counter", f"glm:rank_failures_total {getattr(m, 'rank_failures_total', 0)}",
    ]
    for key, sec in m.phase_seconds.items():
        phase, b = key.split("/b")
        lab = f'{{phase="{phase}",batch_size="{b}"}}'
        lines += [f"glm:phase_seconds_total{lab} {sec}", f"glm:phase_count_total{lab} {m.phase_count.get(key, 0)}"]
    return "\n".join(lines) + "\n"


def normalize_messages(messages: List[dict]) -> List[dict]:
    """What the chat template expects: `content` is never null, and the `arguments` of an assistant message's tool calls
    are objects (clients send them as JSON strings).  Reference: `normalizeMessages` (`src/openai-server.ts:174-194`)."""
    out = []
    for m in messages:
        m = dict(m)
        if m.get("content") is None:
            m["content"] = ""
        calls = m.get("tool_calls")
        if calls:
            fixed = []
            for c in calls:
                c = dict(c)
                fn = dict(c.get("function") or {})
                if isinstance(fn.get("arguments"), str):
                    try:
                        fn["arguments"] = json.loads(fn["arguments"])
                    except ValueError:
                        raise HttpError(400, "tool call arguments must contain valid JSON", param="messages")
                c["function"] = fn
                fixed.append(c)
            m["tool_calls"] = fixed
        out.append(m)
    return out


class OpenAIServer:
    READ_TIMEOUT_S = 30.0            # for the request head and for its body
    MAX_BODY_BYTES = 64 << 20

    def __init__(self, scheduler: GenerationScheduler, tokenizer, cfg: EngineConfig, model_name: str = "glm",
                 max_model_len: int = 65536, healthy=lambda: True, log=None):
        self.sched = scheduler
        self.tok = tokenizer
        self.cfg = cfg
        self.model_name = model_name
        self.max_model_len = max_model_len
        self.healthy = healthy
        self.log = log                    # callable(str) for the per-request performance line, or None
        self.control = resolve_control_tokens(tokenizer)
        self.pending = 0
        self._server: Optional[asyncio.AbstractServer] = None

    # ---- plumbing ---------------------------------------------------------------------------------------
    async def start(self) -> None:
        self._server = await asyncio.start_server(self._client, self.cfg.host, self.cfg.port)

    @property
    def port(self) -> int:
        return self._server.sockets[0].getsockname()[1]

    async def close(self) -> None:
        if self._server:
            self._server.close()
            await self._server.wait_closed()

    async def _client(self, reader: asyncio.StreamReader, writer: asyncio.StreamWriter) -> None:
        try:
            # a client that never finishes its request must not hold a connection for ever
            head = await asyncio.wait_for(reader.readuntil(b"\r\n\r\n"), self.READ_TIMEOUT_S)
            lines = head.decode("latin1").split("\r\n")
            method, path, _ = lines[0].split(" ", 2)
            headers = {}
            for ln in lines[1:]:
                if ":" in ln:
                    k, v = ln.split(":", 1)
                    headers[k.strip().lower()] = v.strip()
            n = int(headers.get("content-length", "0") or 0)
            if n > self.MAX_BODY_BYTES:
                self._send(writer, 413, HttpError(413, f"request body of {n} bytes exceeds {self.MAX_BODY_BYTES}").body())
                await writer.drain()
                return
            body = await asyncio.wait_for(reader.readexactly(n), self.READ_TIMEOUT_S) if n else b""
            await self._route(method, path.split("?")[0], headers, body, writer)
        except (asyncio.IncompleteReadError, asyncio.LimitOverrunError, asyncio.TimeoutError, ConnectionError, ValueError):
            pass
        finally:
            try:
                writer.close()
            except Exception:  # noqa: BLE001
                pass

    @staticmethod
    def _send(writer, status: int, body, ctype="application/json", extra: Optional[Dict[str, str]] = None) -> None:
        data = body if isinstance(body, (bytes, bytearray)) else (json.dumps(body) if not isinstance(body, str) else body).encode()
        reason = {200: "OK", 204: "No Content", 400: "Bad Request", 401: "Unauthorized", 403: "Forbidden", 404: "Not Found",
                  405: "Method Not Allowed", 413: "Payload Too Large", 500: "Internal Server Error", 503: "Service Unavailable"}.get(status, "OK")
        hdr = {"Content-Type": ctype, "Content-Length": str(len(data)), "Connection": "close", **CORS, **(extra or {})}
        writer.write((f"HTTP/1.1 {status} {reason}\r\n" + "".join(f"{k}: {v}\r\n" for k, v in hdr.items()) + "\r\n").encode() + data)

    def _auth(self, headers, admin: bool = False) -> None:
        key = self.cfg.admin_api_key if admin else self.cfg.api_key
        if admin and not key:
            raise HttpError(403, "admin endpoints need --admin-api-key", "permission_error")
        if key and headers.get("authorization", "") != f"Bearer {key}":
            raise HttpError(401, "invalid or missing API key", "authentication_error", param="Authorization", code="invalid_api_key")

    async def _route(self, method, path, headers, body, writer) -> None:
        try:
            if method == "OPTIONS":
                return self._send(writer, 204, b"")
            if method == "GET" and path == "/health":
                ok = self.healthy()
                body = {"status": "ok" if ok else "unhealthy"}
                state = getattr(getattr(self.healthy, "__self__", None), "state", None)      # a HealthMonitor's bound method
                if not ok and state is not None:
                    body.update(reason=state.reason, failed_ranks=list(state.failed_ranks))
                return self._send(writer, 200 if ok else 503, body)
            if method == "GET" and path == "/version":
                return self._send(writer, 200, {"version": __version__})
            if method == "GET" and path == "/metrics":
                txt = render_metrics(self.sched.metrics, self.pending, self.sched.engine.kv, self.cfg.batch_size,
                                     self.cfg.chunk_size, self.max_model_len)
                return self._send(writer, 200, txt, "text/plain; version=0.0.4; charset=utf-8")
            if method == "GET" and path == "/v1/models":
                self._auth(headers)
                return self._send(writer, 200, {"object": "list", "data": [{"id": self.model_name, "object": "model",
                                                                              "owned_by": "slopllm_b200",
                                                                              "max_model_len": self.max_model_len}]})
            if method == "POST" and path == "/tokenize":
                self._auth(headers)
                params = json.loads(body or b"{}")
                ids = self._tokenize(params)
                return self._send(writer, 200, {"tokens": ids, "count": len(ids), "max_model_len": self.max_model_len})
            if method == "POST" and path in ("/admin/flush_gpu_cache", "/admin/flush_host_cache"):
                self._auth(headers, admin=True)
                ev = self.sched.flush_gpu_cache() if path.endswith("gpu_cache") else self.sched.flush_host_cache()
                await asyncio.get_running_loop().run_in_executor(None, ev.done.wait, 60)
                return self._send(writer, 200, ev.result)
            if method == "POST" and path == "/v1/chat/completions":
                self._auth(headers)
                return await self._chat(json.loads(body or b"{}"), writer)
            raise HttpError(404, f"no route {method} {path}", "not_found")
        except HttpError as e:
            self._send(writer, e.status, e.body())
        except json.JSONDecodeError:
            self._send(writer, 400, HttpError(400, "request body is not valid JSON").body())
        except Exception as e:  # noqa: BLE001
            self._send(writer, 500, HttpError(500, f"{type(e).__name__}: {e}", "server_error").body())
        finally:
            try:
                await writer.drain()
            except ConnectionError:
                pass

    # ---- request preparation ----------------------------------------------------------------------------------
    def _tokenize(self, params: dict, kwargs: Optional[dict] = None) -> List[int]:
        if "messages" in params:
            kw = dict(params.get("chat_template_kwargs") or {})
            kw.update(kwargs or {})
            cont = bool(kw.pop("continue_final_message", False))
            ids = self.tok.apply_chat_template(params["messages"], tokenize=True, add_generation_prompt=not cont,
                                               continue_final_message=cont, tools=params.get("tools"), **kw)
            ids = list(ids["input_ids"] if isinstance(ids, dict) else ids)
            if env_flag("CHAT_DEBUG"):      # the rendered prompt as the model sees it (reference: SLOPLLM_CHAT_DEBUG)
                import sys
                print(f"[chat] {len(ids)} prompt tokens:\n{self.tok.decode(ids)}", file=sys.stderr, flush=True)
            return ids
        return list(self.tok.encode(params.get("prompt", ""), add_special_tokens=False))

    def _sampling(self, p: dict) -> SamplingParams:
        d = self.cfg.sampling

        def num(name, default, alias=None):
            v = p.get(name, p.get(alias) if alias else None)
            v = default if v is None else v
            if not isinstance(v, (int, float)) or v != v or v in (float("inf"), float("-inf")):
                raise HttpError(400, f"{name} must be a finite number", param=name)
            return v
        sp = SamplingParams(temperature=max(0.0, float(num("temperature", d.temperature))), top_p=float(num("top_p", d.top_p)),
                            top_k=int(num("top_k", d.top_k)),
                            repetition_penalty=float(num("repetition_penalty", d.repetition_penalty, "frequency_penalty")),
                            presence_penalty=float(num("presence_penalty", d.presence_penalty)),
                            repetition_penalty_window=d.repetition_penalty_window)
        if self.cfg.mtp > 0:
            if sp.top_k > 256:
                raise HttpError(400, "Linear MTP supports top_k <= 256", param="top_k")
            if sp.repetition_penalty != 1 or sp.presence_penalty != 0:
                raise HttpError(400, "MTP decoding currently requires repetition_penalty=1 and presence_penalty=0")
        return sp

    def _parser(self, kwargs: dict) -> ChatModelParser:
        if self.control is None:
            return ChatModelParser(lambda ids: self.tok.decode(list(ids)))
        think = not kwargs.get("continue_final_message") and starts_in_reasoning(
            lambda: self.tok.apply_chat_template([{"role": "user", "content": "Hello"}], tokenize=False,
                                                 add_generation_prompt=True,
                                                 **{k: v for k, v in kwargs.items() if k != "continue_final_message"}))
        return GlmParser(lambda ids: self.tok.decode(list(ids)), self.control, think)

    def _log_request(self, req: GenerationRequest) -> None:
        """One line per finished request: prompt / cached / prefilled tokens, prefill and decode rates (the reference's
        `logRequestPerformance`, `src/openai-server.ts:242-256`).  `log=None` at construction silences it."""
        if self.log is None:
            return
        decoded = max(0, len(req.generated) - 1)
        decode_s = (time.time() - req.first_token_at) if req.first_token_at else 0.0
        prefill_tps = req.prefill_tokens / req.prefill_seconds if req.prefill_seconds > 0 else 0.0
        decode_tps = decoded / decode_s if decode_s > 0 else 0.0
        self.log(f"Request {req.id}: prompt_tokens={req.prompt_tokens} cached_tokens={req.cached_tokens} "
                 f"prefill_tokens={req.prefill_tokens} prefill_tokens_per_second={prefill_tps:.1f} "
                 f"output_tokens={len(req.generated)} decode_tokens_per_second={decode_tps:.1f} finish={req.finish_reason}")

    # ---- chat completions ------------------------------------------------------------------------------------------
    async def _chat(self, params: dict, writer) -> None:
        if not isinstance(params, dict):
            raise HttpError(400, "the request body must be a JSON object")
        if params.get("model") is not None and params["model"] != self.model_name:
            raise HttpError(404, f"The model '{params['model']}' does not exist", param="model", code="model_not_found")
        messages = params.get("messages")
        if not isinstance(messages, list) or not messages or not all(isinstance(m, dict) for m in messages):
            raise HttpError(400, "messages must be a non-empty array of objects", param="messages")
        params = dict(params, messages=normalize_messages(messages))
        messages = params["messages"]
        if params.get("tools") is not None and not isinstance(params["tools"], list):
            raise HttpError(400, "tools must be an array", param="tools")
        if params.get("chat_template_kwargs") is not None and not isinstance(params["chat_template_kwargs"], dict):
            raise HttpError(400, "chat_template_kwargs must be an object", param="chat_template_kwargs")
        kwargs = dict(params.get("chat_template_kwargs") or {})
        # top-level spellings of the two template switches (the request field wins over chat_template_kwargs)
        if params.get("continue_final_message") is not None:
            kwargs["continue_final_message"] = bool(params["continue_final_message"])
        if params.get("enable_thinking") is not None:
            if not isinstance(params["enable_thinking"], bool):
                raise HttpError(400, "enable_thinking must be a boolean", param="enable_thinking")
            kwargs["enable_thinking"] = params["enable_thinking"]
        effort = params.get("reasoning_effort") or env_str("REASONING_EFFORT")      # request field, else the server default
        if effort:
            kwargs.setdefault("reasoning_effort", effort)
        sp = self._sampling(params)
        stops = params.get("stop") or []
        stops = [stops] if isinstance(stops, str) else [s for s in stops if isinstance(s, str)]
        try:
            ids = self._tokenize(params, kwargs)
            parser = self._parser(kwargs)
            if kwargs.get("continue_final_message"):
                parser.continue_from(self.tok.encode(messages[-1].get("content") or "", add_special_tokens=False))
        except HttpError:
            raise
        except Exception as e:  # noqa: BLE001
            raise HttpError(400, f"unable to prepare chat prompt: {e}")
        if len(ids) >= self.max_model_len:
            # (the reference drops the oldest prompt tokens here, `src/openai-server.ts:704-707`; an explicit error lets the
            # client decide what to cut)
            raise HttpError(400, f"prompt has {len(ids)} tokens, the model context is {self.max_model_len}", param="messages",
                            code="context_length_exceeded")
        max_tokens = params.get("max_tokens") or params.get("max_completion_tokens") or self.cfg.max_tokens
        max_tokens = max(1, min(int(max_tokens), self.max_model_len - len(ids)))
        stream = params.get("stream") is True
        stream_options = params.get("stream_options") if isinstance(params.get("stream_options"), dict) else {}
        include_usage = bool(stream_options.get("include_usage"))
        continuous_usage = stream_options.get("continuous_usage_stats") is True      # usage in every streamed chunk

        loop = asyncio.get_running_loop()
        q: asyncio.Queue = asyncio.Queue()
        req = GenerationRequest(id="chatcmpl-" + uuid.uuid4().hex[:24], input_ids=ids, max_tokens=max_tokens, sampling=sp,
                                on_token=lambda t: loop.call_soon_threadsafe(q.put_nowait, ("tok", t)),
                                on_finish=lambda r: loop.call_soon_threadsafe(q.put_nowait, ("end", r)))
        created = int(time.time())
        self.pending += 1
        self.sched.submit(req)
        state = {"content": "", "sent": 0, "reasoning": "", "tools": [], "stopped": False, "ntok": 0}

        def held_back(text: str) -> int:
            """Length of the longest tail of `text` that could still grow into a stop string."""
            best = 0
            for s_ in stops:
                for k in range(min(len(s_) - 1, len(text)), 0, -1):
                    if text.endswith(s_[:k]):
                        best = max(best, k)
                        break
            return best

        def chunk(delta: dict, finish=None, usage=None) -> bytes:
            obj = {"id": req.id, "object": "chat.completion.chunk", "created": created, "model": self.model_name,
                   "choices": [{"index": 0, "delta": delta, "finish_reason": finish}]}
            if usage is None and continuous_usage:
                usage = stream_usage()
            if usage is not None:
                obj["usage"] = usage
            return b"data: " + json.dumps(obj).encode() + b"\n\n"

        def stream_usage() -> dict:
            n = state["ntok"]                              # tokens delivered to this response so far
            return {"prompt_tokens": req.prompt_tokens or len(ids), "completion_tokens": n,
                    "total_tokens": (req.prompt_tokens or len(ids)) + n}

        def usage_obj() -> dict:
            return {"prompt_tokens": req.prompt_tokens, "completion_tokens": len(req.generated),
                    "total_tokens": req.prompt_tokens + len(req.generated),
                    "prompt_tokens_details": {"cached_tokens": req.cached_tokens}}

        def apply(events) -> List[dict]:
            deltas = []
            for ev in events:
                if ev.type == "content_delta":
                    text, hit = check_stop_sequences(state["content"] + ev.text, stops)
                    state["content"] = text
                    upto = len(text) if hit else len(text) - held_back(text)
                    if upto > state["sent"]:
                        deltas.append({"content": text[state["sent"]:upto]})
                        state["sent"] = upto
                    if hit:
                        state["stopped"] = True
                        break
                elif ev.type == "reasoning_delta":
                    state["reasoning"] += ev.text
                    deltas.append({"reasoning_content": ev.text})
                elif ev.type == "tool_call":
                    call = {"index": ev.index, "id": "call_" + uuid.uuid4().hex[:24], "type": "function",
                            "function": {"name": ev.name, "arguments": ev.arguments}}
                    state["tools"].append(call)
                    deltas.append({"tool_calls": [call]})
                elif ev.type == "parse_error":
                    state["content"] += ev.raw
                    deltas.append({"content": state["content"][state["sent"]:]})
                    state["sent"] = len(state["content"])
            return deltas

        try:
            if stream:
                hdr = {"Content-Type": "text/event-stream", "Cache-Control": "no-cache", "Connection": "close",
                       "X-Accel-Buffering": "no", **CORS}             # reverse proxies must not buffer the event stream
                writer.write(("HTTP/1.1 200 OK\r\n" + "".join(f"{k}: {v}\r\n" for k, v in hdr.items()) + "\r\n").encode())
                writer.write(chunk({"role": "assistant", "content": ""}))
            final: Optional[GenerationRequest] = None
            while final is None:
                kind, val = await q.get()
                if kind == "end":
                    final = val
                    events = parser.finish() if not state["stopped"] else []
                else:
                    state["ntok"] += 1
                    events = parser.on_token(val) if not state["stopped"] else []
                deltas = apply(events)
                if kind == "end" and not state["stopped"] and state["sent"] < len(state["content"]):
                    deltas.append({"content": state["content"][state["sent"]:]})      # text held for a stop string that never came
                    state["sent"] = len(state["content"])
                if state["stopped"] and not req.cancelled:
                    # stop string hit.  Only the client-side flag is set from this thread: the scheduler retires the row
                    # (finish reason "stop") in the step in which every rank has learnt of it
                    req.cancel(reason="stop")
                if stream:
                    for d in deltas:
                        writer.write(chunk(d))
                    if continuous_usage and not deltas and kind != "end":
                        # a token that produced no visible text (inside a tool call, a held-back stop prefix) still counts
                        obj = {"id": req.id, "object": "chat.completion.chunk", "created": created, "model": self.model_name,
                               "choices": [], "usage": stream_usage()}
                        writer.write(b"data: " + json.dumps(obj).encode() + b"\n\n")
                    try:
                        await writer.drain()
                    except ConnectionError:
                        req.cancel()                      # client went away
                        return
            self._log_request(req)
            if final.error and not state["stopped"]:
                raise HttpError(500, final.error, "server_error")
            finish = "tool_calls" if parser.produced_tool_calls else ("stop" if state["stopped"] else final.finish_reason or "stop")
            if finish == "cancelled":
                finish = "stop"
            if stream:
                writer.write(chunk({}, finish))
                if include_usage:
                    obj = {"id": req.id, "object": "chat.completion.chunk", "created": created, "model": self.model_name,
                           "choices": [], "usage": usage_obj()}
                    writer.write(b"data: " + json.dumps(obj).encode() + b"\n\n")
                writer.write(b"data: [DONE]\n\n")
            else:
                msg = {"role": "assistant", "content": state["content"] or None}
                if state["reasoning"]:
                    msg["reasoning_content"] = state["reasoning"]
                if state["tools"]:
                    msg["tool_calls"] = [{k: v for k, v in c.items() if k != "index"} for c in state["tools"]]
                self._send(writer, 200, {"id": req.id, "object": "chat.completion", "created": created, "model": self.model_name,
                                         "choices": [{"index": 0, "message": msg, "finish_reason": finish}],
                                         "usage": usage_obj()})
        except HttpError as e:
            if stream:
                writer.write(b"data: " + json.dumps(e.body()).encode() + b"\n\ndata: [DONE]\n\n")
            else:
                raise
        finally:
            self.pending -= 1


async def serve(server: OpenAIServer) -> None:
    await server.start()
    await asyncio.Event().wait()
