"""Python mirror of spbitnet::Tokenizer (reference include/spbitnet/tokenizer.h) over the C-ABI tokenizer, and of
spbitnet::Model::load (include/spbitnet/model.h) over the C++ directory loader."""
from __future__ import annotations

import ctypes as C

import numpy as np

from ._lib import ModelConfig, SpbError, check, load


class Tokenizer:
    """Byte-level BPE over a HuggingFace tokenizer.json; encode adds no BOS / EOS, decode skips special tokens."""

    def __init__(self, tokenizer_json_path):
        self._lib = load()
        self._h = self._lib.spb_tokenizer_load(str(tokenizer_json_path).encode())
        if not self._h:
            raise SpbError(-1, self._lib.spb_last_error_string().decode("utf-8", "replace"))

    @classmethod
    def load(cls, path):
        return cls(path)

    @property
    def vocab_size(self) -> int:
        return self._lib.spb_tokenizer_vocab_size(self._h)

    def encode(self, text) -> list[int]:
        raw = text.encode("utf-8") if isinstance(text, str) else bytes(text)
        n = self._lib.spb_tokenizer_encode(self._h, raw, len(raw), None, 0)
        if n < 0:
            check(n)
        ids = np.zeros(max(n, 1), np.int32)
        self._lib.spb_tokenizer_encode(self._h, raw, len(raw), C.c_void_p(ids.ctypes.data), n)
        return [int(i) for i in ids[:n]]

    def decode_bytes(self, ids) -> bytes:
        a = np.ascontiguousarray(ids, np.int32)
        n = self._lib.spb_tokenizer_decode(self._h, C.c_void_p(a.ctypes.data), a.size, None, 0)
        if n < 0:
            check(n)
        buf = C.create_string_buffer(n + 1)
        self._lib.spb_tokenizer_decode(self._h, C.c_void_p(a.ctypes.data), a.size, buf, n + 1)
        return buf.raw[:n]

    def decode(self, ids) -> str:
        return self.decode_bytes(ids).decode("utf-8", "replace")

    def decode_token(self, token_id: int) -> str:
        return self.decode([int(token_id)])

    def close(self):
        if getattr(self, "_h", None):
            self._lib.spb_tokenizer_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class LoadedModel:
    """A model directory loaded by the C++ loader into one device allocation (current CUDA device)."""

    def __init__(self, model_dir):
        self._lib = load()
        self._h = self._lib.spb_model_load(str(model_dir).encode())
        if not self._h:
            raise SpbError(-5, self._lib.spb_last_error_string().decode("utf-8", "replace"))
        cfg, bos, eos = ModelConfig(), C.c_int(0), C.c_int(0)
        check(self._lib.spb_model_get_config(self._h, C.byref(cfg), C.byref(bos), C.byref(eos)))
        self.config = {name: getattr(cfg, name) for name, _ in ModelConfig._fields_}
        self._cfg, self.bos_token_id, self.eos_token_id = cfg, bos.value, eos.value
        self.device_bytes = self._lib.spb_model_device_bytes(self._h)

    def engine_handle(self):
        """A new C engine with every tensor attached; the caller destroys it with spb_engine_destroy."""
        e = self._lib.spb_engine_create(C.byref(self._cfg))
        if not e:
            raise SpbError(-2, self._lib.spb_last_error_string().decode())
        check(self._lib.spb_model_attach(self._h, e))
        return e

    def close(self):
        if getattr(self, "_h", None):
            self._lib.spb_model_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
