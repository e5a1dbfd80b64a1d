"""OpenAI server over a fake engine: SSE streaming, usage, reasoning / tool-call parsing, stop
strings, auth, /metrics, /tokenize, admin flush.  Parser behaviours mirror the reference's
`tests/test_glm_parser.ts` and `tests/test_incremental_decoder.ts`."""
import asyncio
import json

from slopllm_b200.config import EngineConfig
from slopllm_b200.kv.paged import PagedKVCache
from slopllm_b200.scheduler.scheduler import GenerationScheduler
from slopllm_b200.server.openai import OpenAIServer
from slopllm_b200.server.parsers import GlmParser, IncrementalDecoder, check_stop_sequences, resolve_control_tokens
from slopllm_b200.server.tokenizer import ByteTokenizer


class ScriptEngine:
    """Emits a fixed token script regardless of the prompt."""

    def __init__(self, script):
        self.kv = PagedKVCache(64)
        self.mtp = 0
        self.script = list(script)
        self.pos = {}

    def prefill(self, seqs, prompts, chunk_size=8192, want_hidden=False, rows=None, limits=None):
        out = []
        for s, p in zip(seqs, prompts):
            self.kv.append_tokens(s, p[s.length:])
            self.kv.report_tokens(s)
            self.pos[s.seq_id] = 1
            out.append(self.script[0])
        return out, None

    def decode_step(self, seqs, last, rows=None):
        out = []
        for s, t in zip(seqs, last):
            self.kv.append_tokens(s, [t])
            self.kv.report_tokens(s)
            i = self.pos[s.seq_id]
            self.pos[s.seq_id] = i + 1
            out.append(self.script[min(i, len(self.script) - 1)])
        return out


def test_incremental_decoder_holds_partial_utf8():
    tok = ByteTokenizer()
    dec = IncrementalDecoder(lambda ids: tok.decode(list(ids)))
    ids = tok.encode("héllo ✓")
    out = [dec.push(t) for t in ids]
    assert "".join(out) + dec.flush() == "héllo ✓"
    assert all("�" not in o for o in out)


def test_glm_parser_reasoning_tool_call_and_errors():
    tok = ByteTokenizer()
    ctl = resolve_control_tokens(tok)
    p = GlmParser(lambda ids: tok.decode(list(ids)), ctl, starts_in_reasoning=True)
    text = ("let me think</think>Hello!<tool_call>get_weather\n<arg_key>city</arg_key>\n<arg_value>\"Paris\"</arg_value>\n"
            "<arg_key>days</arg_key><arg_value>3</arg_value></tool_call><tool_call><arg_key>x</arg_key></tool_call>")
    events = []
    for t in tok.encode(text):
        events += p.on_token(t)
    events += p.finish()
    reasoning = "".join(e.text for e in events if e.type == "reasoning_delta")
    content = "".join(e.text for e in events if e.type == "content_delta")
    calls = [e for e in events if e.type == "tool_call"]
    errs = [e for e in events if e.type == "parse_error"]
    assert reasoning == "let me think" and content == "Hello!"
    assert len(calls) == 1 and calls[0].name == "get_weather"
    assert json.loads(calls[0].arguments) == {"city": "Paris", "days": 3}
    assert len(errs) == 1 and "no function name" in errs[0].message
    assert check_stop_sequences("abc STOP def", ["STOP", "def"]) == ("abc ", True)


async def _http(port, method, path, body=None, headers=None):
    r, w = await asyncio.open_connection("127.0.0.1", port)
    data = json.dumps(body).encode() if body is not None else b""
    h = {"Host": "x", "Content-Length": str(len(data)), **(headers or {})}
    w.write((f"{method} {path} HTTP/1.1\r\n" + "".join(f"{k}: {v}\r\n" for k, v in h.items()) + "\r\n").encode() + data)
    await w.drain()
    raw = await r.read()
    w.close()
    head, _, payload = raw.partition(b"\r\n\r\n")
    return int(head.split()[1]), payload


def test_server_endpoints():
    tok = ByteTokenizer()
    script = tok.encode("hm</think>Hi there STOP never<tool_call>f<arg_key>a</arg_key><arg_value>1</arg_value></tool_call>") + [tok.eos_token_id]
    eng = ScriptEngine(script)
    cfg = EngineConfig(host="127.0.0.1", port=0, api_key="k", admin_api_key="adm", batch_size=2, chunk_size=256)
    sched = GenerationScheduler(eng, max_batch=2, chunk_size=256, eos_token_ids=[tok.eos_token_id])
    sched.start()

    async def run():
        lines = []
        srv = OpenAIServer(sched, tok, cfg, model_name="test-model", max_model_len=4096, log=lines.append)
        await srv.start()
        port = srv.port
        auth = {"Authorization": "Bearer k"}
        st, body = await _http(port, "GET", "/health")
        assert st == 200
        st, body = await _http(port, "GET", "/v1/models")
        assert st == 401
        st, body = await _http(port, "GET", "/v1/models", headers=auth)
        assert json.loads(body)["data"][0]["id"] == "test-model"
        st, body = await _http(port, "POST", "/tokenize", {"prompt": "abc"}, auth)
        assert json.loads(body)["tokens"] == [97, 98, 99]
        # non-streaming: reasoning + content + tool call
        st, body = await _http(port, "POST", "/v1/chat/completions",
                               {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 200, "temperature": 0}, auth)
        out = json.loads(body)
        msg = out["choices"][0]["message"]
        assert st == 200 and msg["reasoning_content"] == "hm" and msg["content"] == "Hi there STOP never"
        assert msg["tool_calls"][0]["function"] == {"name": "f", "arguments": '{"a": 1}'}
        assert out["choices"][0]["finish_reason"] == "tool_calls" and out["usage"]["completion_tokens"] == len(script)
        # streaming with a stop string and usage
        st, body = await _http(port, "POST", "/v1/chat/completions",
                               {"messages": [{"role": "user", "content": "hi"}], "stream": True, "stop": ["STOP"],
                                "stream_options": {"include_usage": True}}, auth)
        chunks = [json.loads(l[6:]) for l in body.decode().split("\n\n") if l.startswith("data: {")]
        text = "".join(c["choices"][0]["delta"].get("content", "") for c in chunks if c["choices"])
        assert text == "Hi there " and body.decode().rstrip().endswith("data: [DONE]")
        assert [c for c in chunks if c["choices"] and c["choices"][0]["finish_reason"]][0]["choices"][0]["finish_reason"] == "stop"
        assert any("usage" in c and not c["choices"] for c in chunks)
        assert chunks[0]["choices"][0]["delta"] == {"role": "assistant", "content": ""} and "usage" not in chunks[0]
        # usage in every chunk on request
        st, body = await _http(port, "POST", "/v1/chat/completions",
                               {"messages": [{"role": "user", "content": "hi"}], "stream": True, "max_tokens": 6,
                                "stream_options": {"continuous_usage_stats": True}}, auth)
        cont = [json.loads(l[6:]) for l in body.decode().split("\n\n") if l.startswith("data: {")]
        assert all("usage" in c for c in cont) and cont[-1]["usage"]["completion_tokens"] == 6
        counts = [c["usage"]["completion_tokens"] for c in cont]
        assert counts == sorted(counts) and cont[0]["usage"]["total_tokens"] == cont[0]["usage"]["prompt_tokens"]
        # second identical prompt is served from the prefix cache? (prompt shorter than a page: no) - metrics still count
        st, body = await _http(port, "GET", "/metrics")
        m = body.decode()
        assert "vllm:generation_tokens_total" in m
        assert any(f"vllm:request_success_total {n}" in m for n in (2, 3))         # the stop-string request retires as cancelled
        assert 'vllm:cache_config_info{block_size="64"' in m
        st, body = await _http(port, "POST", "/admin/flush_gpu_cache", {}, auth)
        assert st == 401
        st, body = await _http(port, "POST", "/admin/flush_gpu_cache", {}, {"Authorization": "Bearer adm"})
        assert st == 200 and "gpu_pages_freed" in json.loads(body)
        st, body = await _http(port, "POST", "/v1/chat/completions", {"messages": []}, auth)
        assert st == 400
        # request validation: unknown model, malformed tools / template kwargs / switches, tool-call arguments
        user = [{"role": "user", "content": "x"}]
        st, body = await _http(port, "POST", "/v1/chat/completions", {"model": "other", "messages": user}, auth)
        assert st == 404 and json.loads(body)["error"]["code"] == "model_not_found"
        for bad in ({"tools": {"a": 1}}, {"chat_template_kwargs": [1]}, {"enable_thinking": "yes"}):
            st, body = await _http(port, "POST", "/v1/chat/completions", {"messages": user, **bad}, auth)
            assert st == 400, bad
        call = {"role": "assistant", "content": None, "tool_calls": [{"id": "c1", "type": "function",
                                                                       "function": {"name": "f", "arguments": "{not json"}}]}
        st, body = await _http(port, "POST", "/v1/chat/completions", {"messages": user + [call]}, auth)
        assert st == 400 and "valid JSON" in json.loads(body)["error"]["message"]
        call["tool_calls"][0]["function"]["arguments"] = '{"a": 1}'
        st, body = await _http(port, "POST", "/v1/chat/completions",
                               {"model": "test-model", "messages": user + [call, {"role": "tool", "content": "2"}],
                                "enable_thinking": False, "max_tokens": 4, "temperature": 0}, auth)
        assert st == 200
        st, body = await _http(port, "GET", "/v1/models", headers={"Authorization": "Bearer nope"})
        assert st == 401 and json.loads(body)["error"]["code"] == "invalid_api_key"
        st, body = await _http(port, "POST", "/v1/chat/completions", {"messages": [{"role": "user", "content": "x"}], "top_p": "a"}, auth)
        assert st == 400
        assert len(lines) >= 3 and all("decode_tokens_per_second=" in ln and "prompt_tokens=" in ln for ln in lines)
        # a request that never completes its head is dropped after the read timeout; an oversized body is refused
        srv.READ_TIMEOUT_S = 0.3
        r, w = await asyncio.open_connection("127.0.0.1", port)
        w.write(b"POST /v1/chat/completions HTTP/1.1\r\nHost: x\r\n")          # no blank line
        await w.drain()
        assert await asyncio.wait_for(r.read(), 5) == b""                            # the server closed the connection
        w.close()
        r, w = await asyncio.open_connection("127.0.0.1", port)
        w.write(b"POST /v1/chat/completions HTTP/1.1\r\nHost: x\r\nContent-Length: 999999999999\r\n\r\n")
        await w.drain()
        assert (await asyncio.wait_for(r.read(), 5)).startswith(b"HTTP/1.1 413")
        w.close()
        await srv.close()

    asyncio.run(run())
    sched.stop()


# Model outputs in the GLM protocol, one per shape of response the parser has to take apart (the reference keeps captured
# outputs of the same shapes in `tests/glm_parser_corpus.ts`; these are written for this test).  The opening <think> belongs
# to the prompt, so every output starts inside the reasoning block.
PARSER_CORPUS = [
    {"name": "plain response",
     "output": "The user asks for one word.\n\n1. Output: DONE\n2. Nothing else.</think>DONE",
     "reasoning": "The user asks for one word.\n\n1. Output: DONE\n2. Nothing else.", "content": "DONE", "calls": []},
    {"name": "content followed by a string argument tool call",
     "output": "Need the forecast for Oslo.</think>Let me look that up.<tool_call>get_weather<arg_key>city</arg_key>"
               "<arg_value>Oslo</arg_value></tool_call>",
     "reasoning": "Need the forecast for Oslo.", "content": "Let me look that up.",
     "calls": [("get_weather", {"city": "Oslo"})]},
    {"name": "mixed scalar and array arguments",
     "output": "Timer: 25 minutes, weekdays only, loud.</think>Setting it.<tool_call>set_timer<arg_key>label</arg_key>"
               "<arg_value>focus</arg_value><arg_key>minutes</arg_key><arg_value>25</arg_value><arg_key>days</arg_key>"
               "<arg_value>[\"Mon\", \"Tue\", \"Wed\"]</arg_value><arg_key>volume</arg_key><arg_value>0.8</arg_value>"
               "<arg_key>repeat</arg_key><arg_value>true</arg_value><arg_key>note</arg_key><arg_value>null</arg_value></tool_call>",
     "reasoning": "Timer: 25 minutes, weekdays only, loud.", "content": "Setting it.",
     "calls": [("set_timer", {"label": "focus", "minutes": 25, "days": ["Mon", "Tue", "Wed"], "volume": 0.8, "repeat": True,
                              "note": None})]},
    {"name": "array arguments without visible content",
     "output": "Search both topics.</think><tool_call>search<arg_key>topics</arg_key><arg_value>[\"tcgen05\", \"TMEM\"]"
               "</arg_value><arg_key>limit</arg_key><arg_value>5</arg_value></tool_call>",
     "reasoning": "Search both topics.", "content": "", "calls": [("search", {"topics": ["tcgen05", "TMEM"], "limit": 5})]},
    {"name": "adjacent tool calls",
     "output": "Two cities.</think><tool_call>get_weather<arg_key>city</arg_key><arg_value>Oslo</arg_value></tool_call>"
               "<tool_call>get_weather<arg_key>city</arg_key><arg_value>Lima</arg_value></tool_call>",
     "reasoning": "Two cities.", "content": "", "calls": [("get_weather", {"city": "Oslo"}), ("get_weather", {"city": "Lima"})]},
    {"name": "tool without arguments",
     "output": "Just ask the clock.</think><tool_call>get_time</tool_call>",
     "reasoning": "Just ask the clock.", "content": "", "calls": [("get_time", {})]},
    {"name": "nested object argument with newlines around the markers",
     "output": "Submit the job:\n- name: \"nightly\"\n- retries: 2</think>Submitting.<tool_call>submit_job\n<arg_key>spec</arg_key>\n"
               "<arg_value>{\"name\": \"nightly\", \"retry\": {\"max\": 2, \"backoff\": [1, 5]}, \"tags\": []}</arg_value>\n</tool_call>",
     "reasoning": "Submit the job:\n- name: \"nightly\"\n- retries: 2", "content": "Submitting.",
     "calls": [("submit_job", {"spec": {"name": "nightly", "retry": {"max": 2, "backoff": [1, 5]}, "tags": []}})]},
    {"name": "multi-byte text split across tokens",
     "output": "Grüße – 日本語 ✓</think>Ça marche: “naïve” café 🚀<tool_call>say<arg_key>text</arg_key><arg_value>héllo wörld</arg_value></tool_call>",
     "reasoning": "Grüße – 日本語 ✓", "content": "Ça marche: “naïve” café 🚀", "calls": [("say", {"text": "héllo wörld"})]},
]


def test_glm_parser_corpus_token_by_token():
    """Every corpus entry, fed one token at a time (byte tokens: multi-byte characters arrive in pieces), comes apart into
    exactly its reasoning text, its visible content and its tool calls, with no parse error."""
    tok = ByteTokenizer()
    ctl = resolve_control_tokens(tok)
    for entry in PARSER_CORPUS:
        p = GlmParser(lambda ids: tok.decode(list(ids)), ctl, starts_in_reasoning=True)
        events = []
        for t in tok.encode(entry["output"]):
            events += p.on_token(t)
        events += p.finish()
        assert not [e for e in events if e.type == "parse_error"], entry["name"]
        assert "".join(e.text for e in events if e.type == "reasoning_delta") == entry["reasoning"], entry["name"]
        assert "".join(e.text for e in events if e.type == "content_delta") == entry["content"], entry["name"]
        calls = [(e.name, json.loads(e.arguments)) for e in events if e.type == "tool_call"]
        assert calls == entry["calls"], entry["name"]
        assert [e.index for e in events if e.type == "tool_call"] == list(range(len(calls))), entry["name"]
        assert p.produced_tool_calls == bool(calls)


def test_glm_parser_truncated_tool_call_and_content_mode():
    tok = ByteTokenizer()
    ctl = resolve_control_tokens(tok)
    # generation ends inside a tool call: reported, not silently dropped
    p = GlmParser(lambda ids: tok.decode(list(ids)), ctl, starts_in_reasoning=True)
    events = []
    for t in tok.encode("ok</think>Calling.<tool_call>get_weather<arg_key>city</arg_key><arg_value>Os"):
        events += p.on_token(t)
    events += p.finish()
    assert "".join(e.text for e in events if e.type == "content_delta") == "Calling."
    assert not [e for e in events if e.type == "tool_call"] and [e for e in events if e.type == "parse_error"]
    # thinking disabled by the template: the output starts as content, and a stray </think> never opens reasoning
    p = GlmParser(lambda ids: tok.decode(list(ids)), ctl, starts_in_reasoning=False)
    events = []
    for t in tok.encode("Plain answer."):
        events += p.on_token(t)
    events += p.finish()
    assert "".join(e.text for e in events if e.type == "content_delta") == "Plain answer."
    assert not [e for e in events if e.type == "reasoning_delta"]


def test_parser_continuation_of_an_assistant_prefix():
    """`continue_final_message`: the parser consumes the existing assistant text so that its state (inside or past the
    reasoning block) carries over, and none of the prefix comes back as new output."""
    tok = ByteTokenizer()
    ctl = resolve_control_tokens(tok)
    dec = lambda ids: tok.decode(list(ids))          # noqa: E731
    # the prefix already closed its reasoning: what follows is content
    p = GlmParser(dec, ctl, starts_in_reasoning=False)
    p.continue_from(tok.encode("<think>done thinking</think>The answer is"))
    events = []
    for t in tok.encode(" 42."):
        events += p.on_token(t)
    events += p.finish()
    assert "".join(e.text for e in events if e.type == "content_delta") == " 42."
    assert not [e for e in events if e.type == "reasoning_delta"]
    # the prefix is still inside an open reasoning block: the continuation is reasoning until </think>
    p = GlmParser(dec, ctl, starts_in_reasoning=False)
    p.continue_from(tok.encode("<think>first, consider"))
    events = []
    for t in tok.encode(" the units</think>Metres."):
        events += p.on_token(t)
    events += p.finish()
    assert "".join(e.text for e in events if e.type == "reasoning_delta") == " the units"
    assert "".join(e.text for e in events if e.type == "content_delta") == "Metres."


def test_server_continues_a_partial_assistant_message():
    tok = ByteTokenizer()
    eng = ScriptEngine(tok.encode(" and more.") + [tok.eos_token_id])
    cfg = EngineConfig(host="127.0.0.1", port=0, batch_size=2, chunk_size=256)
    sched = GenerationScheduler(eng, max_batch=2, chunk_size=256, eos_token_ids=[tok.eos_token_id])
    sched.start()

    async def run():
        srv = OpenAIServer(sched, tok, cfg, model_name="m", max_model_len=4096)
        await srv.start()
        msgs = [{"role": "user", "content": "go on"}, {"role": "assistant", "content": "Some text"}]
        for body in ({"messages": msgs, "continue_final_message": True},
                     {"messages": msgs, "chat_template_kwargs": {"continue_final_message": True}}):
            st, raw = await _http(srv.port, "POST", "/v1/chat/completions", {**body, "temperature": 0})
            out = json.loads(raw)
            assert st == 200 and out["choices"][0]["message"]["content"] == " and more."        # the prefix is not repeated
        # the rendered prompt ends with the partial message (no fresh assistant header after it)
        ids = srv._tokenize({"messages": msgs}, {"continue_final_message": True})
        assert tok.decode(ids).endswith("Some text")
        await srv.close()

    asyncio.run(run())
    sched.stop()


def test_broken_tokenizer_is_an_error_not_a_byte_fallback(tmp_path):
    import pytest
    from slopllm_b200.server.tokenizer import load_tokenizer
    assert isinstance(load_tokenizer(str(tmp_path), 300), ByteTokenizer)          # no tokenizer.json: bytes (fixtures)
    (tmp_path / "tokenizer.json").write_text("{ not a tokenizer")
    with pytest.raises(RuntimeError, match="could not be loaded"):
        load_tokenizer(str(tmp_path), 300)
