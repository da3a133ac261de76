"""``Gpt2Tokenizer`` (crates/core/gpu-host/src/tokenizer.rs:34-62): GPT-2's byte-level BPE over a
vocabulary file given at run time (tiktoken's format: one ``base64(token bytes) rank`` pair per line,
as ``r50k_base.tiktoken`` is published; the file itself is data that does not ship with this library).

``encode`` splits the text with GPT-2's pattern using exact Unicode general categories (the ``regex``
module) and merges each piece in the library (``b200nn_bpe_encode_piece``); ``encode_native`` runs the
library's own splitter, which is exact for ASCII text and approximates the categories beyond it.  Both
decode back to the same bytes.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import ERR_SHAPE, NnError, load_library

GPT2_VOCAB_SIZE = 50257
ENDOFTEXT_TOKEN_ID = 50256
ENDOFTEXT = "<|endoftext|>"
GPT2_SPLIT_PATTERN = r"""'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+"""


class TokenizerError(RuntimeError):
    """``TokenizerError::{InitError, DecodeError}`` (tokenizer.rs:14-31)."""


class Gpt2Tokenizer:
    def __init__(self, vocab_path=None, *, ranks: dict | None = None, endoftext_id: int = ENDOFTEXT_TOKEN_ID):
        self.lib = load_library()
        self.endoftext_id = endoftext_id
        self.h = C.c_void_p()
        if ranks is not None:
            toks = list(ranks.items())
            blob = b"".join(t for t, _ in toks)
            offs = np.zeros(len(toks) + 1, dtype=np.uint64)
            offs[1:] = np.cumsum([len(t) for t, _ in toks])
            rk = np.asarray([r for _, r in toks], dtype=np.uint32)
            rc = self.lib.b200nn_bpe_create(blob, offs.ctypes.data_as(C.POINTER(C.c_size_t)),
                                            rk.ctypes.data_as(C.POINTER(C.c_uint32)), len(toks), endoftext_id, C.byref(self.h))
        elif vocab_path is not None:
            rc = self.lib.b200nn_bpe_load(str(vocab_path).encode(), endoftext_id, C.byref(self.h))
        else:
            raise TokenizerError("tokenizer init error: a vocabulary file (tiktoken format) or a rank table is needed")
        if rc != 0:
            raise TokenizerError("tokenizer init error: " + (self.lib.b200nn_bpe_last_error() or b"").decode())
        self._split = None

    def _ids(self, fn, data: bytes):
        cap = max(16, len(data) + 1)
        out = np.empty(cap, dtype=np.uint32)
        n = C.c_size_t()
        rc = fn(self.h, data, len(data), out.ctypes.data_as(C.POINTER(C.c_uint32)), cap, C.byref(n))
        if rc != 0:
            raise TokenizerError((self.lib.b200nn_bpe_last_error() or b"").decode())
        return out[: n.value].tolist()

    def encode_native(self, text: str) -> list:
        """``encode`` with the library's own splitter (what a host without Unicode tables gets)."""
        return self._ids(self.lib.b200nn_bpe_encode, text.encode("utf-8"))

    def encode(self, text: str) -> list:
        """``Gpt2Tokenizer::encode`` = ``encode_with_special_tokens`` (tokenizer.rs:45-47)."""
        if self._split is None:
            import regex
            self._split = regex.compile(GPT2_SPLIT_PATTERN)
        ids = []
        for k, part in enumerate(text.split(ENDOFTEXT)):
            if k:
                ids.append(self.endoftext_id)
            for piece in self._split.findall(part):
                ids += self._ids(self.lib.b200nn_bpe_encode_piece, piece.encode("utf-8"))
        return ids

    def decode_bytes(self, tokens) -> bytes:
        t = np.ascontiguousarray(tokens, dtype=np.uint32)
        n = C.c_size_t()
        p = t.ctypes.data_as(C.POINTER(C.c_uint32))
        rc = self.lib.b200nn_bpe_decode(self.h, p, t.size, None, 0, C.byref(n))
        if rc not in (0, ERR_SHAPE):
            raise TokenizerError("tokenizer decode error: " + (self.lib.b200nn_bpe_last_error() or b"").decode())
        buf = C.create_string_buffer(max(1, n.value))
        rc = self.lib.b200nn_bpe_decode(self.h, p, t.size, buf, n.value, C.byref(n))
        if rc != 0:
            raise TokenizerError("tokenizer decode error: " + (self.lib.b200nn_bpe_last_error() or b"").decode())
        return buf.raw[: n.value]

    def decode(self, tokens) -> str:
        """``Gpt2Tokenizer::decode`` (tokenizer.rs:50-55): fails when the bytes are not UTF-8."""
        try:
            return self.decode_bytes(tokens).decode("utf-8")
        except UnicodeDecodeError as e:
            raise TokenizerError(f"tokenizer decode error: {e}") from e

    def vocab_size(self) -> int:
        """The size of the loaded table including the special token (50257 for r50k_base)."""
        return int(self.lib.b200nn_bpe_vocab_size(self.h))

    def __del__(self):
        try:
            if self.h:
                self.lib.b200nn_bpe_destroy(self.h)
        except Exception:
            pass
