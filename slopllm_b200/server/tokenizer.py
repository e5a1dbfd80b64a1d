"""Tokenizer + chat template access.

The reference vendors `@huggingface/transformers` (`src/chat_model.ts:701-724`); here the Python
`transformers` tokenizer of the model directory is used when present.  `ByteTokenizer` is the
self-contained stand-in for tests and for synthetic-weight servers without tokenizer files.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Sequence


class ByteTokenizer:
    """UTF-8 bytes as ids 0..255 plus structural tokens; a fixed, simple chat template."""

    SPECIAL = ["<|system|>", "<|user|>", "<|assistant|>", "<|observation|>", "<think>", "</think>", "<tool_call>",
               "</tool_call>", "<|endoftext|>"]

    def __init__(self, vocab_size: int = 512):
        self.vocab_size = vocab_size
        self.special: Dict[str, int] = {t: 256 + i for i, t in enumerate(self.SPECIAL)}
        self.inv = {v: k for k, v in self.special.items()}
        self.eos_token_id = self.special["<|endoftext|>"]
        self.unk_token_id = -1

    def convert_tokens_to_ids(self, tok: str) -> int:
        return self.special.get(tok, -1)

    def encode(self, text: str, add_special_tokens: bool = False) -> List[int]:
        out: List[int] = []
        i = 0
        while i < len(text):
            for sp, sid in self.special.items():
                if text.startswith(sp, i):
                    out.append(sid)
                    i += len(sp)
                    break
            else:
                out.extend(text[i].encode("utf-8"))
                i += 1
        return out

    def decode(self, ids: Sequence[int], skip_special_tokens: bool = False) -> str:
        buf = bytearray()
        parts: List[str] = []
        for t in ids:
            if 0 <= t < 256:
                buf.append(t)
            else:
                if buf:
                    parts.append(buf.decode("utf-8", errors="replace"))
                    buf = bytearray()
                if not skip_special_tokens and t in self.inv:
                    parts.append(self.inv[t])
        if buf:
            parts.append(buf.decode("utf-8", errors="replace"))
        return "".join(parts)

    def apply_chat_template(self, messages, tokenize=True, add_generation_prompt=True, enable_thinking=True,
                            continue_final_message=False, tools=None, **_):
        text = ""
        if tools:
            import json
            text += "<|system|>\n# Tools\n" + "\n".join(json.dumps(t, ensure_ascii=False) for t in tools)
        for i, m in enumerate(messages):
            role = m.get("role", "user")
            tag = {"system": "<|system|>", "user": "<|user|>", "assistant": "<|assistant|>", "tool": "<|observation|>"}.get(role, "<|user|>")
            content = m.get("content") or ""
            if isinstance(content, list):
                content = "".join(p.get("text", "") for p in content if isinstance(p, dict))
            text += f"{tag}\n{content}"
        if continue_final_message:
            pass
        elif add_generation_prompt:
            text += "<|assistant|>\n" + ("<think>" if enable_thinking else "<think></think>")
        return self.encode(text) if tokenize else text


def load_tokenizer(model_dir: Optional[str], vocab_size: int = 512):
    """The Hugging Face tokenizer of `model_dir` (or of SLOPLLM_B200_TOKENIZER_REPO).  The byte tokenizer is only for
    directories without a `tokenizer.json` (random-init models, test fixtures): a checkpoint whose tokenizer exists but
    cannot be loaded is an error, not a reason to serve bytes."""
    from ..config import env_str
    path = env_str("TOKENIZER_REPO") or model_dir
    if path and os.path.exists(os.path.join(path, "tokenizer.json")):
        try:
            from transformers import AutoTokenizer
            return AutoTokenizer.from_pretrained(path, local_files_only=True)
        except Exception as e:  # noqa: BLE001
            raise RuntimeError(f"{path} has a tokenizer.json but it could not be loaded: {type(e).__name__}: {e}") from e
    return ByteTokenizer(vocab_size)
