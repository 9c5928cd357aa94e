"""Tokenizer access.  A local HF tokenizer directory is used when the model path has one;
random-weight runs fall back to a byte-level tokenizer (ids 0..255 + BOS/EOS) so that the text
API, streaming detokenisation and the chat template path stay exercisable offline."""
from __future__ import annotations

import os


class ByteTokenizer:
    bos_token_id, eos_token_id, pad_token_id = 256, 257, 258
    vocab_size = 259

    def encode(self, text: str, add_special_tokens: bool = False, special: dict | None = None) -> list[int]:
        """``special``: marker string -> token id (a model's chat and placeholder tokens); markers found in the text
        become their one id, everything between them is encoded byte by byte."""
        if special:
            import re
            ids = []
            for part in re.split("(" + "|".join(re.escape(k) for k in sorted(special, key=len, reverse=True)) + ")", text):
                if part in special:
                    ids.append(int(special[part]))
                elif part:
                    ids.extend(part.encode("utf-8"))
        else:
            ids = list(text.encode("utf-8"))
        return ([self.bos_token_id] + ids) if add_special_tokens else ids

    def decode(self, ids, skip_special_tokens: bool = True) -> str:
        b = bytes(i for i in ids if 0 <= i < 256)
        return b.decode("utf-8", errors="replace")

    def apply_chat_template(self, messages, add_generation_prompt=True, tokenize=False, **_):
        parts = []
        for m in messages:
            c = m.get("content")
            if isinstance(c, list):
                c = "".join(p.get("text", "") for p in c if isinstance(p, dict) and p.get("type") == "text")
            parts.append(f"<|im_start|>{m.get('role', 'user')}\n{c or ''}<|im_end|>\n")
        if add_generation_prompt:
            parts.append("<|im_start|>assistant\n")
        text = "".join(parts)
        return self.encode(text) if tokenize else text


def get_tokenizer(model: str | None, trust_remote_code: bool = False):
    if model and os.path.isdir(model) and any(os.path.exists(os.path.join(model, f))
                                              for f in ("tokenizer.json", "tokenizer_config.json", "vocab.json")):
        from transformers import AutoTokenizer
        return AutoTokenizer.from_pretrained(model, trust_remote_code=trust_remote_code, local_files_only=True)
    return ByteTokenizer()


class IncrementalDetokenizer:
    """Streams text for a growing token list without re-decoding the whole sequence each step
    and without emitting half of a multi-byte character."""

    def __init__(self, tokenizer, skip_special_tokens: bool = True):
        self.tok, self.skip = tokenizer, skip_special_tokens
        self.ids: list[int] = []
        self.prefix_len = 0       # tokens whose text is final
        self.text = ""

    def add(self, new_ids: list[int]) -> str:
        self.ids.extend(new_ids)
        window = self.ids[self.prefix_len:]
        piece = self.tok.decode(window, skip_special_tokens=self.skip)
        if piece.endswith("�"):          # incomplete UTF-8 sequence: wait for more tokens
            return ""
        self.prefix_len = len(self.ids)
        self.text += piece
        return piece
