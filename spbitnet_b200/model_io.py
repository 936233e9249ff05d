"""Model directory I/O in the reference's on-disk format (docs/compression_format.md section 4,
written by python/convert_model.py, read by Model::load, src/model.cu:179-311).

    <dir>/config.json              architecture parameters
    <dir>/manifest.json            {"format_version": 1, "weights": {name: entry}}
    <dir>/weights/<name>.meta|.values|.bin    raw little-endian row-major arrays

`load_model_dir` returns the host model layout that `spbitnet_b200.synth.random_model` produces and
`spbitnet_b200.engine.DeviceModel` uploads; `save_model_dir` writes that layout, so a directory made
by the reference's converter and one made here are interchangeable.  Sparse tensors are checked on
load (sizes against shape and strides, every bitmap exactly two bits) because the kernels assume it.
"""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np

from . import _lib
from .synth import LINEAR_NAMES, NORM_NAMES

FORMAT_VERSION = 1
_LINEAR_PREFIX = ["self_attn", "self_attn", "self_attn", "self_attn", "mlp", "mlp", "mlp"]
_NORM_PREFIX = ["", "", "self_attn.", "mlp."]
_CONFIG_DEFAULTS = {"model_type": "bitnet", "hidden_act": "relu2", "tie_word_embeddings": True}


class ModelFormatError(ValueError):
    """The directory does not follow the format (missing entry, wrong size, invalid bitmap)."""


def _linear_name(layer: int, i: int) -> str:
    return f"layers.{layer}.{_LINEAR_PREFIX[i]}.{LINEAR_NAMES[i]}"


def _norm_name(layer: int, i: int) -> str:
    return f"layers.{layer}.{_NORM_PREFIX[i]}{NORM_NAMES[i]}"


def save_model_dir(model: dict, path, stats: bool = False) -> Path:
    """Writes `model` (random_model layout) as a model directory.  Returns the directory."""
    root = Path(path)
    (root / "weights").mkdir(parents=True, exist_ok=True)
    cfg = dict(_CONFIG_DEFAULTS)
    cfg.update(model["config"])
    tied = "lm_head" not in model or model["lm_head"] is None
    cfg["tie_word_embeddings"] = bool(tied)
    (root / "config.json").write_text(json.dumps(cfg, indent=2))
    weights = {}

    def dense(name: str, arr: np.ndarray, dtype: str):
        rel = f"weights/{name}.bin"
        np.ascontiguousarray(arr).tofile(root / rel)
        weights[name] = {"file": rel, "dtype": dtype, "shape": list(arr.shape), "nbytes": int(arr.nbytes)}

    dense("embed_tokens", model["embed"].astype(np.float16, copy=False), "float16")
    dense("norm", model["final_norm"].astype(np.float32, copy=False), "float32")
    if tied:
        weights["lm_head"] = {"tied_to": "embed_tokens", "dtype": "tied"}
    else:
        dense("lm_head", model["lm_head"].astype(np.float16, copy=False), "float16")
    for l, layer in enumerate(model["layers"]):
        for i, t in enumerate(layer["linear"]):
            name = _linear_name(l, i)
            meta = np.ascontiguousarray(t["meta"], dtype=np.uint32)
            values = np.ascontiguousarray(t["values"], dtype=np.uint32)
            meta.tofile(root / f"weights/{name}.meta")
            values.tofile(root / f"weights/{name}.values")
            entry = {"meta_file": f"weights/{name}.meta", "values_file": f"weights/{name}.values",
                     "dtype": "sparse_ternary", "shape": [int(t["rows"]), int(t["cols"])],
                     "meta_stride": int(meta.shape[1]), "values_stride": int(values.shape[1]),
                     "gamma": float(t["gamma"]), "meta_nbytes": int(meta.nbytes), "values_nbytes": int(values.nbytes)}
            if stats:
                nz = int(t["rows"]) * int(t["cols"]) // 2
                entry["stats"] = {"nz_after_pruning": nz, "density_after": 0.5}
            weights[name] = entry
        for i, n in enumerate(layer["norm"]):
            if n is not None:
                dense(_norm_name(l, i), np.asarray(n, dtype=np.float32), "float32")
    (root / "manifest.json").write_text(json.dumps({"format_version": FORMAT_VERSION, "weights": weights}, indent=1))
    return root


def _read(root: Path, rel: str, dtype, count: int, what: str) -> np.ndarray:
    f = root / rel
    if not f.is_file():
        raise ModelFormatError(f"{what}: file {rel} is missing")
    want = count * np.dtype(dtype).itemsize
    if f.stat().st_size != want:
        raise ModelFormatError(f"{what}: {rel} has {f.stat().st_size} bytes, expected {want}")
    return np.fromfile(f, dtype=dtype, count=count)


def load_model_dir(path, validate: bool = True, layers: int | None = None) -> dict:
    """Reads a model directory into the host layout of `random_model`.  `layers` limits the depth."""
    root = Path(path)
    try:
        cfg = json.loads((root / "config.json").read_text())
        manifest = json.loads((root / "manifest.json").read_text())
    except FileNotFoundError as exc:
        raise ModelFormatError(f"{root}: {exc.filename} is missing") from None
    if manifest.get("format_version") != FORMAT_VERSION:
        raise ModelFormatError(f"format_version {manifest.get('format_version')!r} is not {FORMAT_VERSION}")
    weights = manifest.get("weights", {})
    for key in ("hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "intermediate_size",
                "vocab_size", "max_position_embeddings", "rms_norm_eps", "rope_theta"):
        if key not in cfg:
            raise ModelFormatError(f"config.json: field {key} is missing")
    cfg.setdefault("head_dim", cfg["hidden_size"] // cfg["num_attention_heads"])
    L = cfg["num_hidden_layers"] if layers is None else min(layers, cfg["num_hidden_layers"])

    def entry(name: str, required: bool = True):
        e = weights.get(name)
        if e is None and required:
            raise ModelFormatError(f"manifest.json: no entry {name}")
        return e

    def dense(name: str, dtype, required: bool = True):
        e = entry(name, required)
        if e is None:
            return None
        if e.get("dtype") != np.dtype(dtype).name:
            raise ModelFormatError(f"{name}: dtype {e.get('dtype')!r}, expected {np.dtype(dtype).name}")
        shape = tuple(int(s) for s in e["shape"])
        return _read(root, e["file"], dtype, int(np.prod(shape)), name).reshape(shape)

    model = {"config": dict(cfg, num_hidden_layers=L), "layers": []}
    model["embed"] = dense("embed_tokens", np.float16)
    model["final_norm"] = dense("norm", np.float32)
    head = weights.get("lm_head")
    if head is not None and head.get("dtype") != "tied":
        model["lm_head"] = dense("lm_head", np.float16)
    lib = _lib.load() if validate else None
    for l in range(L):
        layer = {"linear": [], "norm": []}
        for i in range(len(LINEAR_NAMES)):
            name = _linear_name(l, i)
            e = entry(name)
            if e.get("dtype") != "sparse_ternary":
                raise ModelFormatError(f"{name}: dtype {e.get('dtype')!r}, expected sparse_ternary")
            rows, cols = (int(s) for s in e["shape"])
            ms, vs = int(e["meta_stride"]), int(e["values_stride"])
            if cols % 4 or ms < (cols // 4 + 7) // 8 or vs < (cols // 4 + 15) // 16:
                raise ModelFormatError(f"{name}: shape {rows}x{cols} does not fit strides {ms}/{vs}")
            meta = _read(root, e["meta_file"], np.uint32, rows * ms, name).reshape(rows, ms)
            values = _read(root, e["values_file"], np.uint32, rows * vs, name).reshape(rows, vs)
            if validate:
                import ctypes as C
                rc = lib.spb_validate_packed(meta.ctypes.data_as(C.c_void_p), rows, cols, ms)
                if rc != 0:
                    raise ModelFormatError(f"{name}: {lib.spb_last_error_string().decode()}")
            layer["linear"].append({"meta": meta, "values": values, "gamma": np.float32(e["gamma"]), "rows": rows,
                                    "cols": cols, "meta_stride": ms, "values_stride": vs})
        for i in range(len(NORM_NAMES)):
            layer["norm"].append(dense(_norm_name(l, i), np.float32, required=i < 2))
        model["layers"].append(layer)
    return model
