"""Tokenizer access for the HTTP frontend: chat templates, incremental detokenisation,
stop-string matching.

In the reference these live in the external Rust frontend it launches
(``src/parallax/server/vllm_rust_frontend.py:85-136``); here they are part of the package.
When a checkpoint directory has tokenizer files, the HuggingFace tokenizer is used. For
random-init models without tokenizer files a byte-level fallback keeps the HTTP surface
usable (ids 0..255 are bytes, 256 = BOS, 257 = EOS).
"""

from __future__ import annotations

import logging
import os
from typing import Optional

logger = logging.getLogger(__name__)

DEFAULT_CHAT_TEMPLATE = (
    "{% for m in messages %}<|im_start|>{{ m['role'] }}\n{{ m['content'] }}<|im_end|>\n{% endfor %}"
    "{% if add_generation_prompt %}<|im_start|>assistant\n{% endif %}"
)


class ByteTokenizer:
    """Byte-level stand-in used when no tokenizer files are available."""

    bos_token_id, eos_token_id = 256, 257
    vocab_size = 258
    chat_template = DEFAULT_CHAT_TEMPLATE

    def encode(self, text: str, add_special_tokens: bool = False) -> list[int]:
        ids = list(text.encode("utf-8"))
        return ([self.bos_token_id] + ids) if add_special_tokens else ids

    def decode(self, ids, skip_special_tokens: bool = True) -> str:
        return bytes(i for i in ids if 0 <= i < 256).decode("utf-8", errors="replace")


class TokenizerWrapper:
    def __init__(self, tokenizer=None, vocab_size: Optional[int] = None):
        self.tok = tokenizer or ByteTokenizer()
        self.vocab_size = vocab_size or getattr(self.tok, "vocab_size", None)

    @classmethod
    def from_pretrained(cls, model_path: Optional[str], vocab_size: Optional[int] = None) -> "TokenizerWrapper":
        if model_path and os.path.isdir(model_path) and any(
                os.path.exists(os.path.join(model_path, f)) for f in ("tokenizer.json", "tokenizer.model",
                                                                       "tokenizer_config.json")):
            from transformers import AutoTokenizer

            return cls(AutoTokenizer.from_pretrained(model_path, trust_remote_code=False), vocab_size)
        if model_path and not os.path.isdir(model_path):
            try:
                from transformers import AutoTokenizer

                return cls(AutoTokenizer.from_pretrained(model_path, local_files_only=True), vocab_size)
            except Exception as e:
                logger.warning("tokenizer of %s unavailable (%s); using the byte-level fallback", model_path, e)
        return cls(None, vocab_size)

    @property
    def eos_token_ids(self) -> set[int]:
        e = getattr(self.tok, "eos_token_id", None)
        if e is None:
            return set()
        return {int(x) for x in e} if isinstance(e, (list, tuple)) else {int(e)}

    def encode(self, text: str, add_special_tokens: bool = True) -> list[int]:
        ids = list(self.tok.encode(text, add_special_tokens=add_special_tokens))
        return self._clamp(ids)

    def decode(self, ids, skip_special_tokens: bool = True) -> str:
        return self.tok.decode(list(ids), skip_special_tokens=skip_special_tokens)

    def token_text(self, token_id: int) -> Optional[str]:
        """Text that this token adds on its own, or None for special tokens and for tokens that are only a
        fragment of a character (constrained decoding checks candidate tokens with this)."""
        cache = self.__dict__.setdefault("_token_text", {})
        if token_id in cache:
            return cache[token_id]
        t: Optional[str]
        if isinstance(self.tok, ByteTokenizer):
            t = chr(token_id) if token_id < 128 else None
        else:
            try:
                t = self.tok.decode([int(token_id)], skip_special_tokens=True)
            except Exception:
                t = None
            if t is not None and (t == "" or "\ufffd" in t):
                t = None
        cache[token_id] = t
        return t

    def _clamp(self, ids: list[int]) -> list[int]:
        # random-init models may have a smaller vocabulary than the tokenizer in use
        if self.vocab_size:
            return [i % self.vocab_size for i in ids]
        return ids

    def apply_chat_template(self, messages: list[dict], add_generation_prompt: bool = True, **kw) -> list[int]:
        if hasattr(self.tok, "apply_chat_template") and getattr(self.tok, "chat_template", None):
            out = self.tok.apply_chat_template(messages, tokenize=True, add_generation_prompt=add_generation_prompt, **kw)
            if isinstance(out, dict):
                out = out["input_ids"]
            return self._clamp(list(out))
        import jinja2

        text = jinja2.Template(getattr(self.tok, "chat_template", None) or DEFAULT_CHAT_TEMPLATE).render(
            messages=[{"role": m.get("role", "user"), "content": _content_text(m.get("content"))} for m in messages],
            add_generation_prompt=add_generation_prompt)
        return self.encode(text, add_special_tokens=False)


class LazyTokenizer:
    """A :class:`TokenizerWrapper` that is loaded at first use: ranks of a multi-process engine that never
    sample a constrained request never pay for reading the vocabulary."""

    def __init__(self, model_path: Optional[str], vocab_size: Optional[int] = None):
        self._args = (model_path, vocab_size)
        self._tok: Optional[TokenizerWrapper] = None

    def __getattr__(self, name):
        if name.startswith("_"):
            raise AttributeError(name)
        if self._tok is None:
            self._tok = TokenizerWrapper.from_pretrained(*self._args)
        return getattr(self._tok, name)


def _content_text(content) -> str:
    if isinstance(content, str):
        return content
    if isinstance(content, list):  # OpenAI content parts
        return "".join(p.get("text", "") for p in content if isinstance(p, dict) and p.get("type", "text") == "text")
    return "" if content is None else str(content)


class IncrementalDetokenizer:
    """Streams text for a growing token sequence without re-emitting or splitting characters.

    Decodes a sliding window (``prefix_offset`` .. end) and emits only text that no longer ends
    in an incomplete UTF-8 sequence; holds back text that could be the start of a stop string.
    """

    def __init__(self, tokenizer: TokenizerWrapper, stop: Optional[list[str]] = None, skip_special_tokens: bool = True):
        self.t = tokenizer
        self.stop = [s for s in (stop or []) if s]
        self.skip_special = skip_special_tokens
        self.ids: list[int] = []
        self.prefix_offset = 0
        self.read_offset = 0
        self.text = ""          # everything decoded so far
        self.emitted = 0        # characters already handed out
        self.stopped = False
        self._hold = max((len(s) for s in self.stop), default=1) - 1

    def add(self, token_id: int) -> str:
        """Feed one token; returns the new text that may be shown to the client."""
        if self.stopped:
            return ""
        self.ids.append(int(token_id))
        prefix = self.t.decode(self.ids[self.prefix_offset:self.read_offset], self.skip_special)
        full = self.t.decode(self.ids[self.prefix_offset:], self.skip_special)
        if len(full) > len(prefix) and not full.endswith("�"):
            self.text += full[len(prefix):]
            self.prefix_offset = self.read_offset
            self.read_offset = len(self.ids)
        return self._release(final=False)

    def _release(self, final: bool) -> str:
        for s in self.stop:
            i = self.text.find(s, max(0, self.emitted - len(s)))
            if i != -1:
                self.stopped = True
                out = self.text[self.emitted:i]
                self.text = self.text[:i]
                self.emitted = len(self.text)
                return out
        upto = len(self.text) if final else max(self.emitted, len(self.text) - self._hold)
        out = self.text[self.emitted:upto]
        self.emitted = upto
        return out

    def flush(self) -> str:
        return "" if self.stopped else self._release(final=True)
