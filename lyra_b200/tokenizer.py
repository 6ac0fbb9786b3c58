"""Tokenizer: tiktoken ``o200k_base`` extended with the Harmony special tokens -> ``o200k_harmony``
(lyra/tokenizer.py:6-55). eos = 199999, pad = 200004, vocabulary padded to 204,800.

tiktoken fetches the ``o200k_base`` merge table on first use. Where that is impossible (no network and no
``TIKTOKEN_CACHE_DIR`` / ``LYRA_O200K_PATH`` file) the class falls back to a byte-level vocabulary with the same
special-token ids, so sampling, serving and the tests still run; ``LyraTokenizer().is_fallback`` says which one is active.
"""

from __future__ import annotations

import os

PADDED_VOCAB_SIZE = 204800

_HARMONY_SPECIALS = {
    "<|startoftext|>": 199998, "<|endoftext|>": 199999, "<|reserved_200000|>": 200000, "<|reserved_200001|>": 200001,
    "<|return|>": 200002, "<|constrain|>": 200003, "<|reserved_200004|>": 200004, "<|channel|>": 200005,
    "<|start|>": 200006, "<|end|>": 200007, "<|message|>": 200008, "<|reserved_200009|>": 200009,
    "<|reserved_200010|>": 200010, "<|reserved_200011|>": 200011, "<|call|>": 200012,
}
_O200K_BASE_SPECIALS = {"<|endoftext|>": 199999, "<|endofprompt|>": 200018}


def _load_base():
    import tiktoken

    local = os.environ.get("LYRA_O200K_PATH")
    if local and os.path.exists(local):
        from tiktoken.load import load_tiktoken_bpe

        pat = "|".join([
            r"[^\r\n\p{L}\p{N}]?[\p{Lu}\p{Lt}\p{Lm}\p{Lo}\p{M}]*[\p{Ll}\p{Lm}\p{Lo}\p{M}]+(?i:'s|'t|'re|'ve|'m|'ll|'d)?",
            r"[^\r\n\p{L}\p{N}]?[\p{Lu}\p{Lt}\p{Lm}\p{Lo}\p{M}]+[\p{Ll}\p{Lm}\p{Lo}\p{M}]*(?i:'s|'t|'re|'ve|'m|'ll|'d)?",
            r"\p{N}{1,3}", r" ?[^\s\p{L}\p{N}]+[\r\n/]*", r"\s*[\r\n]+", r"\s+(?!\S)", r"\s+",
        ])
        return tiktoken.Encoding(name="o200k_base", pat_str=pat, mergeable_ranks=load_tiktoken_bpe(local),
                                 special_tokens=dict(_O200K_BASE_SPECIALS))
    return tiktoken.get_encoding("o200k_base")


class _ByteEncoding:
    """Offline stand-in: UTF-8 bytes are token ids 0..255; special tokens keep their real ids."""

    def __init__(self, specials: dict[str, int]):
        self._specials = specials
        self._by_id = {v: k for k, v in specials.items()}

    def encode_ordinary(self, text: str) -> list[int]:
        return list(text.encode("utf-8"))

    def encode(self, text: str) -> list[int]:
        return self.encode_ordinary(text)

    def encode_ordinary_batch(self, texts, num_threads: int = 8):
        return [self.encode_ordinary(t) for t in texts]

    def decode_single_token_bytes(self, token: int) -> bytes:
        if token < 256:
            return bytes([token])
        return self._by_id.get(token, "").encode("utf-8")

    def decode(self, tokens) -> str:
        return b"".join(self.decode_single_token_bytes(int(t)) for t in tokens).decode("utf-8", errors="replace")


class LyraTokenizer:
    def __init__(self):
        self.is_fallback = False
        try:
            import tiktoken

            base = _load_base()
            self._special_tokens = {**base._special_tokens, **_HARMONY_SPECIALS} | {
                f"<|reserved_{i}|>": i for i in range(200013, PADDED_VOCAB_SIZE) if i not in base._special_tokens.values()
            }
            self.tokenizer = tiktoken.Encoding(name="o200k_harmony", pat_str=base._pat_str, mergeable_ranks=base._mergeable_ranks,
                                               special_tokens=self._special_tokens)
        except Exception:
            self.is_fallback = True
            self._special_tokens = {**_O200K_BASE_SPECIALS, **_HARMONY_SPECIALS} | {
                f"<|reserved_{i}|>": i for i in range(200013, PADDED_VOCAB_SIZE) if i not in _O200K_BASE_SPECIALS.values()
            }
            self.tokenizer = _ByteEncoding(self._special_tokens)

    def encode(self, text: str) -> list[int]:
        return self.tokenizer.encode(text)

    def encode_ordinary(self, text: str) -> list[int]:
        return self.tokenizer.encode_ordinary(text)

    def encode_ordinary_batch(self, texts: list[str], num_threads: int = 8) -> list[list[int]]:
        return self.tokenizer.encode_ordinary_batch(texts, num_threads=num_threads)

    def decode(self, tokens: list[int]) -> str:
        return self.tokenizer.decode(tokens)

    def decode_single_token_bytes(self, token: int) -> bytes:
        return self.tokenizer.decode_single_token_bytes(token)

    @property
    def eos_token(self) -> int:
        return self._special_tokens["<|endoftext|>"]

    @property
    def pad_token(self) -> int:
        return self._special_tokens["<|reserved_200004|>"]
