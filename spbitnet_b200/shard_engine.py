"""Python host of the row-sharded engine (spb_shard_engine_* of the C-ABI): one instance per rank, one process
per GPU.  It cuts a full model into the rank's row slices, uploads them, exchanges the CUDA IPC handles of the
exchange buffers over torch.distributed and drives the engine.  The reference is single-GPU
(include/spbitnet/inference.h:23-70); forward/generate/reset mirror its InferenceEngine and greedy loop
(src/main.cpp:266-300) for `batch` sequences in lock step."""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from ._lib import ModelConfig, SpbError, check, load

_CFG_KEYS = ["hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "head_dim",
             "intermediate_size", "vocab_size", "max_position_embeddings", "rms_norm_eps", "rope_theta"]


class ShardEngine:
    """model: a device model with FULL weights in the layout of spbitnet_b200.engine.DeviceModel /
    synth.DeviceRandomModel (this rank keeps contiguous copies of its row slices only; the caller may drop the
    full model afterwards).  With world > 1 a torch.distributed process group (any backend) must be
    initialised: it carries the 64-byte IPC handles and the barriers, never activations."""

    def __init__(self, model, rank: int = 0, world: int = 1, batch: int = 1, group=None, timeout_ms: int | None = None,
                 connect: bool = True):
        self._lib = load()
        self.rank, self.world, self.batch, self.group = rank, world, batch, group
        self.config = dict(model.config)
        cfg = ModelConfig(**{k: self.config[k] for k in _CFG_KEYS})
        self.device = model.device
        with torch.cuda.device(self.device):
            self._h = self._lib.spb_shard_engine_create(C.byref(cfg), rank, world, batch)
        if not self._h:
            raise SpbError(-1, self._lib.spb_last_error_string().decode())
        self._keep = []
        self.ranges = [self.row_range(i) for i in range(8)]
        for l, layer in enumerate(model.layers):
            self.set_layer(l, layer)
        head = model.lm_head if getattr(model, "lm_head", None) is not None else model.embed
        v0, v1 = self.ranges[7]
        head_rows = head[v0:v1].clone()
        self._keep += [model.embed, head_rows, model.final_norm]
        check(self._lib.spb_shard_engine_set_globals(self._h, C.c_void_p(model.embed.data_ptr()),
                                                     C.c_void_p(head_rows.data_ptr()),
                                                     C.c_void_p(model.final_norm.data_ptr())))
        self.vocab_rows = v1 - v0
        if timeout_ms is not None:
            check(self._lib.spb_shard_engine_set_timeout_ms(self._h, int(timeout_ms)))
        if world > 1 and connect:
            self.connect()

    def row_range(self, which: int) -> tuple[int, int]:
        a, b = C.c_int(0), C.c_int(0)
        check(self._lib.spb_shard_engine_row_range(self._h, which, C.byref(a), C.byref(b)))
        return a.value, b.value

    def set_layer(self, l: int, layer: dict, share_from=None) -> None:
        """Attaches the rank's slices of one layer.  layer["linear"][i] holds the FULL matrix (d_meta, d_values as
        CUDA int32 tensors [rows, stride]); a contiguous copy of rows [start, stop) is kept."""
        for i, t in enumerate(layer["linear"]):
            r0, r1 = self.ranges[i]
            # clone(): a row slice of a contiguous matrix is itself contiguous, and layers that alias one host
            # layer must still get separate device storage (every layer streams its own bytes from HBM)
            meta, values = t["d_meta"][r0:r1].clone(), t["d_values"][r0:r1].clone()
            self._keep += [meta, values]
            check(self._lib.spb_shard_engine_set_linear(self._h, l, i, C.c_void_p(meta.data_ptr()),
                                                        C.c_void_p(values.data_ptr()), float(t["gamma"]), r1 - r0,
                                                        t["cols"], t["meta_stride"], t["values_stride"]))
        for i, n in enumerate(layer["norm"]):
            if n is not None:
                self._keep.append(n)
                check(self._lib.spb_shard_engine_set_norm(self._h, l, i, C.c_void_p(n.data_ptr())))

    def connect(self) -> None:
        """Exchanges the IPC handles of the exchange buffers over the process group and maps the peers'."""
        import torch.distributed as dist
        mine = (C.c_ubyte * 64)()
        check(self._lib.spb_shard_engine_ipc_handle(self._h, mine))
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(mine), group=self.group)
        blob = b"".join(handles)
        check(self._lib.spb_shard_engine_set_peers(self._h, C.c_char_p(blob)))
        dist.barrier(group=self.group)  # every rank has mapped every buffer before the first exchange

    def step(self, tokens) -> None:
        """One decode step of all sequences; tokens: `batch` ids.  Every rank must call it with the same ids."""
        t = np.ascontiguousarray(np.atleast_1d(tokens), np.int32)
        assert t.size == self.batch
        check(self._lib.spb_shard_engine_step(self._h, C.c_void_p(t.ctypes.data)))

    def logits_rows(self) -> np.ndarray:
        """This rank's vocabulary rows of the last step's logits: [batch, stop - start] float32."""
        h = np.empty((self.batch, self.vocab_rows), np.float32)
        check(self._lib.spb_shard_engine_copy_logits(self._h, C.c_void_p(h.ctypes.data)))
        return h

    def logits(self) -> np.ndarray:
        """The full logits [batch, vocab] on every rank (rows gathered over the process group on the host)."""
        rows = self.logits_rows()
        if self.world == 1:
            return rows
        import torch.distributed as dist
        parts = [None] * self.world
        dist.all_gather_object(parts, rows, group=self.group)
        return np.concatenate(parts, axis=1)

    def generate(self, prompt, max_tokens: int) -> np.ndarray:
        """prompt: [n_prompt, batch] (or [n_prompt] when batch is 1) token ids; returns [max_tokens, batch]."""
        p = np.ascontiguousarray(prompt, np.int32).reshape(-1, self.batch)
        out = np.zeros((max(max_tokens, 1), self.batch), np.int32)
        n = self._lib.spb_shard_engine_generate(self._h, C.c_void_p(p.ctypes.data), p.shape[0], int(max_tokens),
                                                C.c_void_p(out.ctypes.data))
        if n < 0:
            check(n)
        return out[:n]

    def reset(self) -> None:
        check(self._lib.spb_shard_engine_reset(self._h))

    @property
    def seq_len(self) -> int:
        return self._lib.spb_shard_engine_seq_len(self._h)

    @property
    def exchange_bytes(self) -> int:
        return self._lib.spb_shard_engine_exchange_bytes(self._h)

    def set_peer_pointers(self, pointers) -> None:
        arr = (C.c_void_p * self.world)(*[C.c_void_p(p) for p in pointers])
        check(self._lib.spb_shard_engine_set_peer_pointers(self._h, arr))

    def set_prepared_weights(self, level: int) -> None:
        """Whether the engine multiplies on prepared copies of its slices (kernels.prepare_weights): 1 (default) those
        of 4 M weights and more, 2 every slice the layout takes, 0 none.  Wide models, one sequence; same results either way."""
        check(self._lib.spb_shard_engine_set_prepared_weights(self._h, int(level)))

    def set_exchange_fold(self, form: int) -> None:
        """Wide models, one sequence, several ranks: 2 (default) the producing kernels store their slices into every
        rank's staging area from their epilogues and the consuming kernels poll it, 1 the consuming kernel performs
        the exchange, 0 a launch of its own does.  Same results every way."""
        check(self._lib.spb_shard_engine_set_exchange_fold(self._h, int(form)))

    def weight_bytes(self) -> int:
        """Bytes of weights this rank streams per decode step (its row slices + its LM head rows)."""
        n = sum(t.numel() * t.element_size() for t in self._keep if t.dtype == torch.int32)
        return n + self.vocab_rows * self.config["hidden_size"] * 2

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.spb_shard_engine_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
