"""ctypes binding of the C-ABI declared in include/spbitnet_b200.h.

The library is the product: there is no Python or CPU fallback.  If the shared object
is missing the import fails with instructions to build it.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_HERE = Path(__file__).resolve().parent
LIB_PATH = _HERE / "libspbitnet_b200.so"

SPB_OK = 0
SPB_E_INVALID = -1
SPB_E_CUDA = -2
SPB_E_TIMEOUT = -3
SPB_E_UNSUPPORTED = -4
SPB_E_FORMAT = -5


class SpbError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"spbitnet_b200 error {code}: {message}")
        self.code = code


class ModelConfig(C.Structure):
    """spb_model_config: the ModelConfig fields the forward pass reads
    (reference include/spbitnet/model.h:22-38)."""
    _fields_ = [
        ("hidden_size", C.c_int), ("num_hidden_layers", C.c_int),
        ("num_attention_heads", C.c_int), ("num_key_value_heads", C.c_int),
        ("head_dim", C.c_int), ("intermediate_size", C.c_int), ("vocab_size", C.c_int),
        ("max_position_embeddings", C.c_int), ("rms_norm_eps", C.c_float), ("rope_theta", C.c_float),
    ]


_p = C.c_void_p
_i = C.c_int
_f = C.c_float


class GemvItem(C.Structure):
    """spb_gemv_item: one entry of a GEMV work list."""
    _fields_ = [("meta", C.c_void_p), ("values", C.c_void_p), ("x", C.c_void_p), ("y", C.c_void_p),
                ("rows", C.c_int), ("cols", C.c_int), ("meta_row_stride", C.c_int), ("values_row_stride", C.c_int)]


# name -> (restype, argtypes); every symbol include/spbitnet_b200.h declares.
SIGNATURES = {
    "spb_last_error_string": (C.c_char_p, []),
    "spb_version": (C.c_char_p, []),
    "spb_set_pdl": (_i, [_i]),
    "spb_set_gemv_variant": (_i, [_i]),
    "spb_sparse_ternary_unpack": (_i, [_p, _p, _p, _i, _i, _i, _i, _p]),
    "spb_sparse_ternary_gemv": (_i, [_p, _p, _p, _p, _i, _i, _i, _i, _p]),
    "spb_sparse_ternary_gemv_scaled": (_i, [_p, _p, _p, _p, _p, _p, _f, _i, _i, _i, _i, _p]),
    "spb_fused_sparse_bitlinear": (_i, [_p, _p, _p, _p, _p, _f, _i, _i, _i, _i, _p]),
    "spb_sparse_bitlinear_q8": (_i, [_p, _p, _p, _p, _p, _f, _i, _i, _i, _i, _p]),
    "spb_gemv_batch_check": (_i, [_p, _i]),
    "spb_sparse_ternary_gemv_batch": (_i, [_p, _i, _i, _i, _p]),
    "spb_sparse_ternary_gemm": (_i, [_p, _p, _p, _p, _i, _i, _i, _i, _i, _p]),
    "spb_sparse_bitlinear_gemm": (_i, [_p, _p, _p, _p, _p, C.c_float, _p, _i, _i, _i, _i, _i, _p]),
    "spb_set_gemm_variant": (_i, [_i]),
    "spb_set_gemm_row_halves": (_i, [_i]),
    "spb_gemm_tc_timeouts": (_i, []),
    "spb_prepared_weights_bytes": (C.c_size_t, [_i, _i]),
    "spb_prepare_weights": (_i, [_p, _p, _i, _i, _i, _i, _p, _p]),
    "spb_prepared_gemv": (_i, [_p, _p, _p, _i, _i, _p]),
    "spb_prepared_bitlinear_q8": (_i, [_p, _p, _p, _p, _f, _i, _i, _p]),
    "spb_debug_bounded_wait_selftest": (_i, [C.c_longlong, _p]),
    "spb_debug_grid_barrier_selftest": (_i, [C.c_longlong, _p]),
    "spb_debug_set_decode_trace": (None, [_p]),
    "spb_rms_norm": (_i, [_p, _p, _p, _i, _f, _p]),
    "spb_absmax_quantize": (_i, [_p, _p, _p, _i, _p]),
    "spb_absmax_reduce": (_i, [_p, _p, _i, _p]),
    "spb_dequantize": (_i, [_p, _p, _p, _f, _i, _p]),
    "spb_rope": (_i, [_p, _i, _i, _i, _f, _p]),
    "spb_scatter_kv": (_i, [_p, _p, _i, _i, _i, _i, _p]),
    "spb_attention_scores": (_i, [_p, _p, _p, _i, _i, _i, _i, _i, _f, _p]),
    "spb_softmax": (_i, [_p, _i, _i, _i, _p]),
    "spb_attention_output": (_i, [_p, _p, _p, _i, _i, _i, _i, _i, _p]),
    "spb_relu2_mul": (_i, [_p, _p, _p, _i, _p]),
    "spb_relu2_mul_f32": (_i, [_p, _p, _p, _i, _p]),
    "spb_rms_norm_f32in": (_i, [_p, _p, _p, _i, _f, _p]),
    "spb_float_to_half": (_i, [_p, _p, _i, _p]),
    "spb_residual_add": (_i, [_p, _p, _p, _i, _p]),
    "spb_half_gemv": (_i, [_p, _p, _p, _i, _i, _p]),
    "spb_decode_attention": (_i, [_p, _p, _p, _p, _i, _i, _i, _i, _i, _f, _p]),
    "spb_decode_attention_scratch_bytes": (C.c_size_t, [_i, _i, _i]),
    "spb_decode_attention_split": (_i, [_p, _p, _p, _p, _i, _i, _i, _i, _i, _f, _p, C.c_size_t, _p]),
    "spb_decode_attention_noalloc_capacity": (C.c_size_t, []),
    "spb_decode_attention_noalloc": (_i, [_p, _p, _p, _p, _i, _i, _i, _i, _i, _f, _p]),
    "spb_meta_words_per_row": (_i, [_i]),
    "spb_values_words_per_row": (_i, [_i]),
    "spb_pack_from_dense": (_i, [_p, _p, _i, _i, _p, _p]),
    "spb_pack_with_pruning": (_i, [_p, _i, _i, _p, _p]),
    "spb_unpack_to_int8_host": (_i, [_p, _p, _i, _i, _i, _i, _p]),
    "spb_validate_packed": (_i, [_p, _i, _i, _i]),
    "spb_prune_pack_gpu": (_i, [_p, _i, _i, C.c_size_t, _p, _p, _i, _i, _p, _p]),
    "spb_engine_create": (_p, [C.POINTER(ModelConfig)]),
    "spb_engine_destroy": (None, [_p]),
    "spb_engine_set_linear": (_i, [_p, _i, _i, _p, _p, _f, _i, _i, _i, _i]),
    "spb_engine_set_norm": (_i, [_p, _i, _i, _p]),
    "spb_engine_set_globals": (_i, [_p, _p, _p, _p]),
    "spb_engine_forward": (_i, [_p, _i, C.POINTER(_p)]),
    "spb_engine_reset": (_i, [_p]),
    "spb_engine_seq_len": (_i, [_p]),
    "spb_engine_generate": (_i, [_p, _p, _i, _i, _i, _p]),
    "spb_engine_copy_logits": (_i, [_p, _p]),
    "spb_engine_prefill": (_i, [_p, _p, _i, _p]),
    "spb_engine_set_prefill_chunk": (_i, [_p, _i]),
    "spb_engine_set_decode_mode": (_i, [_p, _i]),
    "spb_engine_set_prepared_weights": (_i, [_p, _i]),
    "spb_engine_decode_is_persistent": (_i, [_p]),
    "spb_model_load": (_p, [C.c_char_p]),
    "spb_model_destroy": (None, [_p]),
    "spb_model_get_config": (_i, [_p, C.POINTER(ModelConfig), C.POINTER(_i), C.POINTER(_i)]),
    "spb_model_device_bytes": (C.c_size_t, [_p]),
    "spb_model_attach": (_i, [_p, _p]),
    "spb_tokenizer_load": (_p, [C.c_char_p]),
    "spb_tokenizer_destroy": (None, [_p]),
    "spb_tokenizer_vocab_size": (_i, [_p]),
    "spb_tokenizer_encode": (_i, [_p, C.c_char_p, C.c_size_t, _p, _i]),
    "spb_tokenizer_decode": (_i, [_p, _p, _i, _p, C.c_size_t]),
    "spb_shard_engine_create": (_p, [C.POINTER(ModelConfig), _i, _i, _i]),
    "spb_shard_engine_destroy": (None, [_p]),
    "spb_shard_engine_row_range": (_i, [_p, _i, C.POINTER(_i), C.POINTER(_i)]),
    "spb_shard_engine_set_linear": (_i, [_p, _i, _i, _p, _p, _f, _i, _i, _i, _i]),
    "spb_shard_engine_set_norm": (_i, [_p, _i, _i, _p]),
    "spb_shard_engine_set_globals": (_i, [_p, _p, _p, _p]),
    "spb_shard_engine_ipc_handle": (_i, [_p, _p]),
    "spb_shard_engine_set_peers": (_i, [_p, _p]),
    "spb_shard_engine_set_peer_pointers": (_i, [_p, _p]),
    "spb_shard_engine_exchange_bytes": (C.c_size_t, [_p]),
    "spb_shard_engine_set_timeout_ms": (_i, [_p, _i]),
    "spb_shard_engine_set_prepared_weights": (_i, [_p, _i]),
    "spb_shard_engine_set_exchange_fold": (_i, [_p, _i]),
    "spb_shard_engine_reset": (_i, [_p]),
    "spb_shard_engine_seq_len": (_i, [_p]),
    "spb_shard_engine_step": (_i, [_p, _p]),
    "spb_shard_engine_copy_logits": (_i, [_p, _p]),
    "spb_shard_engine_generate": (_i, [_p, _p, _i, _i, _p]),
}

_lib = None


def load() -> C.CDLL:
    """Loads the shared library and attaches the signatures.  Raises if it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing. Build it with `python -m spbitnet_b200.build` (needs nvcc); "
            "there is no fallback implementation.")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means header and library disagree
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(status: int) -> None:
    if status != SPB_OK:
        raise SpbError(status, load().spb_last_error_string().decode("utf-8", "replace"))
