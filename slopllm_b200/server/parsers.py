"""Output parsers: incremental detokenisation and the GLM reasoning / tool-call protocol.

Parity: `src/chat-model-parser.ts:1-239` (stateful parser, structural markers handled by token
id, text decoded from a retained token prefix so byte-level fragments are never emitted early),
`src/glm-parser.ts:1-94` (`<think>`, `<tool_call>name<arg_key>k</arg_key><arg_value>v</arg_value>`),
`src/chat-continuation.ts:1-25` (assistant-prefix continuation).
"""
from __future__ import annotations

import json
import re
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence


class IncrementalDecoder:
    """Decode a token stream to text without emitting partial UTF-8 / merge fragments.

    Keeps the ids of the current unflushed tail; text is emitted when decoding the tail no longer
    ends in the replacement character, and only the part that is stable is released.
    """

    def __init__(self, decode: Callable[[Sequence[int]], str], hold: int = 6):
        self._decode = decode
        self._ids: List[int] = []
        self._emitted = ""
        self._hold = hold

    def push(self, token_id: int) -> str:
        self._ids.append(token_id)
        text = self._decode(self._ids)
        if text.endswith("�"):
            return ""                                   # incomplete byte sequence: wait
        new = text[len(self._emitted):]
        self._emitted = text
        if len(self._ids) > 64:                         # bound the retained prefix
            self._ids, self._emitted = [], ""
        return new

    def flush(self) -> str:
        text = self._decode(self._ids) if self._ids else ""
        new = text[len(self._emitted):]
        self._ids, self._emitted = [], ""
        return new


@dataclass
class ParserEvent:
    type: str                     # reasoning_delta | content_delta | tool_call | parse_error
    text: str = ""
    index: int = 0
    name: str = ""
    arguments: str = ""
    message: str = ""
    raw: str = ""


@dataclass
class ControlTokens:
    think_start: int
    think_end: int
    tool_call_start: int
    tool_call_end: int


class ChatModelParser:
    """Base parser: without control tokens everything is content."""

    def __init__(self, decode: Callable[[Sequence[int]], str], control: Optional[ControlTokens] = None,
                 state: str = "content"):
        self._decode_ids = decode
        self.control = control
        self.state = state
        self._text = IncrementalDecoder(decode)
        self._tool_ids: List[int] = []
        self._tool_index = 0
        self.produced_tool_calls = False

    # -- hooks ---------------------------------------------------------------------------------------
    def parse_tool_call(self, raw: str) -> Dict[str, object]:
        raise NotImplementedError

    # -- stream ---------------------------------------------------------------------------------------
    def _text_event(self, text: str) -> ParserEvent:
        return ParserEvent("reasoning_delta" if self.state == "reasoning" else "content_delta", text=text)

    def _flush_text(self) -> List[ParserEvent]:
        t = self._text.flush()
        return [self._text_event(t)] if t else []

    def continue_from(self, token_ids: Sequence[int]) -> None:
        """Consume an existing assistant prefix (continuation of a partial message)."""
        for t in token_ids:
            self.on_token(t)
        self._flush_text()

    def on_token(self, token_id: int) -> List[ParserEvent]:
        c = self.control
        if c is None:
            t = self._text.push(token_id)
            return [ParserEvent("content_delta", text=t)] if t else []
        if self.state == "tool":
            if token_id != c.tool_call_end:
                self._tool_ids.append(token_id)
                return []
            return self._finish_tool()
        if token_id == c.think_start:
            ev = self._flush_text()
            self.state = "reasoning"
            return ev
        if token_id == c.think_end:
            ev = self._flush_text()
            self.state = "content"
            return ev
        if token_id == c.tool_call_start:
            ev = self._flush_text()
            self.state = "tool"
            self._tool_ids = []
            return ev
        t = self._text.push(token_id)
        return [self._text_event(t)] if t else []

    def _finish_tool(self) -> List[ParserEvent]:
        raw = self._decode_ids(self._tool_ids)
        self._tool_ids = []
        self.state = "content"
        try:
            call = self.parse_tool_call(raw)
        except ValueError as err:
            return [ParserEvent("parse_error", message=str(err), raw=raw)]
        ev = ParserEvent("tool_call", index=self._tool_index, name=str(call["name"]),
                         arguments=json.dumps(call["arguments"], ensure_ascii=False))
        self._tool_index += 1
        self.produced_tool_calls = True
        return [ev]

    def finish(self) -> List[ParserEvent]:
        """End of generation: an unterminated tool call is parsed as far as it goes."""
        if self.state == "tool":
            return self._finish_tool()
        return self._flush_text()


_ARG = re.compile(r"<arg_key>([\s\S]*?)</arg_key>\s*<arg_value>([\s\S]*?)</arg_value>")


class GlmParser(ChatModelParser):
    """GLM chat-template output protocol.  The generation prompt pre-fills `<think>` when
    thinking is enabled, so the model then starts inside the reasoning block."""

    def __init__(self, decode, control: Optional[ControlTokens], starts_in_reasoning: bool = True):
        super().__init__(decode, control, "reasoning" if (starts_in_reasoning and control) else "content")

    def parse_tool_call(self, raw: str) -> Dict[str, object]:
        first = raw.find("<arg_key>")
        name = (raw if first == -1 else raw[:first]).strip()
        if not name:
            raise ValueError("GLM tool call has no function name")
        args: Dict[str, object] = {}
        n = 0
        for m in _ARG.finditer(raw):
            key = m.group(1).strip()
            if not key:
                raise ValueError("GLM tool call contains an empty argument name")
            val = m.group(2).strip()
            try:
                args[key] = json.loads(val)
            except json.JSONDecodeError:
                args[key] = val
            n += 1
        if first != -1 and n == 0:
            raise ValueError("GLM tool call contains malformed arguments")
        return {"name": name, "arguments": args}


def resolve_control_tokens(tokenizer) -> Optional[ControlTokens]:
    """Look the four structural markers up in the tokenizer's vocabulary (None if any is missing)."""
    ids = []
    for tok in ("<think>", "</think>", "<tool_call>", "</tool_call>"):
        try:
            i = tokenizer.convert_tokens_to_ids(tok)
        except Exception:  # noqa: BLE001
            return None
        if i is None or i < 0 or i == getattr(tokenizer, "unk_token_id", -1):
            return None
        ids.append(int(i))
    return ControlTokens(*ids)


def starts_in_reasoning(render_prompt: Callable[[], str]) -> bool:
    """Probe the rendered generation prompt: does the assistant prefix leave a `<think>` open?"""
    text = render_prompt()
    tail = text[text.rfind("<|assistant|>") + len("<|assistant|>"):] if "<|assistant|>" in text else text
    return tail.rfind("<think>") > tail.rfind("</think>")


def check_stop_sequences(text: str, stops: Sequence[str]):
    """Returns (emit_text, stopped): text up to the earliest stop string."""
    best = -1
    for s in stops:
        if not s:
            continue
        i = text.find(s)
        if i != -1 and (best == -1 or i < best):
            best = i
    if best == -1:
        return text, False
    return text[:best], True
