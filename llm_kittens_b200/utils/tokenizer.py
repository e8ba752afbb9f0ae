"""Token-id -> bytes decoder backed by the C++ tokenizer table (file magic 20240328; reference
llmc/tokenizer.h:25-105)."""
from __future__ import annotations

import ctypes

from . import hostlib


class Tokenizer:
    def __init__(self, path: str):
        self._lib = hostlib.lib()
        self._h = self._lib.llmk_tokenizer_create(path.encode())
        self.init_ok = bool(self._h)
        self.vocab_size = int(self._lib.llmk_tokenizer_vocab_size(self._h)) if self.init_ok else 0
        self.eot_token = int(self._lib.llmk_tokenizer_eot(self._h)) if self.init_ok else 50256

    def close(self):
        if getattr(self, "_h", None):
            self._lib.llmk_tokenizer_destroy(self._h)
            self._h = None

    __del__ = close

    def decode(self, token_id: int) -> bytes | None:
        if not self.init_ok:
            return None
        buf = ctypes.create_string_buffer(256)
        n = self._lib.llmk_tokenizer_decode(self._h, int(token_id), buf, 256)
        if n < 0:
            return None
        return buf.raw[:n]

    @staticmethod
    def safe_text(piece: bytes | None) -> str:
        """Printable rendering: drops lone control bytes like the reference's safe_printf."""
        if not piece:
            return ""
        if len(piece) == 1 and not (32 <= piece[0] < 127 or piece[0] in (9, 10, 13)):
            return ""
        return piece.decode("utf-8", errors="replace")
