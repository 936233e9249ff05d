"""Python mirror of spbitnet::InferenceEngine (reference include/spbitnet/inference.h:23-70)
over the C-ABI engine: forward(token) -> device logits, reset(), seq_len, plus the greedy
loop of src/main.cpp:266-300 as generate()."""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from ._lib import ModelConfig, check, load, SpbError

_CFG_KEYS = ["hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "head_dim",
             "intermediate_size", "vocab_size", "max_position_embeddings", "rms_norm_eps", "rope_theta"]


class DeviceModel:
    """Uploads a host model (spbitnet_b200.synth.random_model layout) to the current CUDA device.
    Plays the part of spbitnet::Model (include/spbitnet/model.h): it owns the weight tensors."""

    def __init__(self, model: dict, device=None):
        self.config = dict(model["config"])
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.device = dev
        self.embed = torch.from_numpy(model["embed"].view(np.int16)).to(dev).view(torch.float16)
        self.final_norm = torch.from_numpy(model["final_norm"]).to(dev)
        head = model.get("lm_head")  # absent or None: tied to the embedding table
        self.lm_head = None if head is None else torch.from_numpy(head.view(np.int16)).to(dev).view(torch.float16)
        self.layers = []
        for layer in model["layers"]:  # every layer gets its own device copy, also when the host arrays are shared
            lin = []
            for t in layer["linear"]:
                meta = torch.from_numpy(t["meta"].view(np.int32)).to(dev)
                values = torch.from_numpy(t["values"].view(np.int32)).to(dev)
                lin.append(dict(t, d_meta=meta, d_values=values))
            norms = [None if n is None else torch.from_numpy(n).to(dev) for n in layer["norm"]]
            self.layers.append({"linear": lin, "norm": norms})

    def sparse_bytes(self) -> int:
        return sum(t["d_meta"].numel() * 4 + t["d_values"].numel() * 4 for L in self.layers for t in L["linear"])


class InferenceEngine:
    def __init__(self, model: DeviceModel, use_sub_norm: bool = True):
        self._lib = load()
        self.model = model
        cfg = ModelConfig(**{k: model.config[k] for k in _CFG_KEYS})
        with torch.cuda.device(model.device):
            self._h = self._lib.spb_engine_create(C.byref(cfg))
        if not self._h:
            raise SpbError(-2, self._lib.spb_last_error_string().decode())
        for l, layer in enumerate(model.layers):
            for i, t in enumerate(layer["linear"]):
                check(self._lib.spb_engine_set_linear(self._h, l, i, C.c_void_p(t["d_meta"].data_ptr()),
                                                      C.c_void_p(t["d_values"].data_ptr()), float(t["gamma"]),
                                                      t["rows"], t["cols"], t["meta_stride"], t["values_stride"]))
            for i, n in enumerate(layer["norm"]):
                if n is None or (i >= 2 and not use_sub_norm):
                    continue
                check(self._lib.spb_engine_set_norm(self._h, l, i, C.c_void_p(n.data_ptr())))
        head = C.c_void_p(model.lm_head.data_ptr() if model.lm_head is not None else 0)
        check(self._lib.spb_engine_set_globals(self._h, C.c_void_p(model.embed.data_ptr()), head,
                                               C.c_void_p(model.final_norm.data_ptr())))

    @classmethod
    def from_loaded(cls, loaded):
        """An engine over a model directory read by the C++ loader (spbitnet_b200.tokenizer.LoadedModel)."""
        self = cls.__new__(cls)
        self._lib = load()
        self.model = loaded
        self._h = loaded.engine_handle()
        return self

    def forward(self, token_id: int) -> int:
        """One token; returns the device address of the logits (vocab_size float32)."""
        out = C.c_void_p(0)
        check(self._lib.spb_engine_forward(self._h, int(token_id), C.byref(out)))
        return out.value

    def prefill(self, tokens) -> int:
        """The tokens as one batch from the current position (what forward() token by token does, with the
        BitLinear layers as the batched product); returns the device address of the last token's logits."""
        t = np.ascontiguousarray(tokens, np.int32)
        out = C.c_void_p(0)
        check(self._lib.spb_engine_prefill(self._h, C.c_void_p(t.ctypes.data), len(t), C.byref(out)))
        return out.value

    def set_prefill_chunk(self, chunk: int) -> int:
        """generate() feeds the prompt token by token when 0 (the reference's loop, default), else in batches
        of up to `chunk` tokens.  Returns the previous setting."""
        prev = self._lib.spb_engine_set_prefill_chunk(self._h, int(chunk))
        if prev < 0:
            check(prev)
        return prev

    DECODE_AUTO, DECODE_CHAIN, DECODE_PERSISTENT, DECODE_UNFUSED, DECODE_PERSISTENT_TAGGED = 0, 1, 2, 3, 4

    def set_decode_mode(self, mode: int) -> None:
        """How the layers of a decode token run: DECODE_AUTO = DECODE_CHAIN (five PDL-linked kernels per layer),
        DECODE_PERSISTENT (one cooperative launch per token, grid barriers between the stages),
        DECODE_PERSISTENT_TAGGED (the same launch without grid barriers: stage outputs travel as tagged words that
        their consumers poll), DECODE_UNFUSED (one launch per op group).
        All modes give the same tokens and logits."""
        check(self._lib.spb_engine_set_decode_mode(self._h, int(mode)))

    def set_prepared_weights(self, on: bool) -> None:
        """Whether the default decode chain multiplies on prepared copies of the matrices (built and owned by the
        engine; default on) or on the packed format.  Same tokens and logits either way."""
        check(self._lib.spb_engine_set_prepared_weights(self._h, int(bool(on))))

    @property
    def decode_is_persistent(self) -> bool:
        return bool(self._lib.spb_engine_decode_is_persistent(self._h))

    def logits(self) -> np.ndarray:
        h = np.empty(self.model.config["vocab_size"], np.float32)
        check(self._lib.spb_engine_copy_logits(self._h, C.c_void_p(h.ctypes.data)))
        return h

    def reset(self) -> None:
        check(self._lib.spb_engine_reset(self._h))

    @property
    def seq_len(self) -> int:
        return self._lib.spb_engine_seq_len(self._h)

    def generate(self, prompt, max_tokens: int, eos_token_id: int = -1) -> np.ndarray:
        p = np.ascontiguousarray(prompt, np.int32)
        out = np.zeros(max(max_tokens, 1), np.int32)
        n = self._lib.spb_engine_generate(self._h, C.c_void_p(p.ctypes.data), len(p), int(max_tokens),
                                          int(eos_token_id), C.c_void_p(out.ctypes.data))
        if n < 0:
            check(n)
        return out[:n]

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.spb_engine_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
