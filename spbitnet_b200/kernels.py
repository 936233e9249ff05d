"""Python mirror of the reference's kernel host wrappers (namespace spbitnet,
include/spbitnet/sparse_ternary_kernels.h and inference_kernels.h): same names, same
argument order, torch CUDA tensors in place of device pointers.  Every function forwards
to the C-ABI of libspbitnet_b200.so; errors raise SpbError instead of exiting.
"""
from __future__ import annotations

import ctypes as C

import torch

from ._lib import check, load


def _p(t):
    if t is None:
        return C.c_void_p(0)
    if isinstance(t, int):
        return C.c_void_p(t)
    return C.c_void_p(t.data_ptr())


def _stream(stream):
    if stream is None:
        return C.c_void_p(torch.cuda.current_stream().cuda_stream)
    if isinstance(stream, int):
        return C.c_void_p(stream)
    return C.c_void_p(stream.cuda_stream)


def set_pdl(enabled: bool) -> bool:
    return bool(load().spb_set_pdl(int(enabled)))


def set_gemv_variant(variant: int) -> int:
    """0 automatic, 1 pair kernel, 2 per-group table kernel, 3 tcgen05 sparse kernel, 4 warp-level sparse MMA kernel."""
    return load().spb_set_gemv_variant(int(variant))


def set_gemm_variant(variant: int) -> int:
    """0 automatic, 1 SIMT form, 2 tcgen05 tensor-core form."""
    return load().spb_set_gemm_variant(int(variant))


def set_gemm_row_halves(halves: int) -> int:
    """0 automatic, 1 / 2 weight-row halves per block of the tcgen05 product; returns the previous setting."""
    return load().spb_set_gemm_row_halves(int(halves))


def gemm_tc_timeouts() -> int:
    return load().spb_gemm_tc_timeouts()


def debug_bounded_wait_selftest(limit_cycles: int = 4000, stream=None) -> int:
    """Runs the library's bounded-wait self-test and returns its status code (SPB_E_TIMEOUT is the
    expected answer: the wait ran out, was counted, and the block returned)."""
    return load().spb_debug_bounded_wait_selftest(int(limit_cycles), _stream(stream))


def debug_grid_barrier_selftest(limit_cycles: int = 200000, stream=None) -> int:
    """Two blocks at a grid barrier of the persistent decode step that expects three arrivals: returns
    SPB_E_TIMEOUT when both bounded waits ran out, were counted and the kernel returned."""
    return load().spb_debug_grid_barrier_selftest(int(limit_cycles), _stream(stream))


# ---- sparse_ternary_kernels.h ---------------------------------------------------------

def sparse_ternary_unpack_gpu(meta, values, out, rows, cols, meta_row_stride, values_row_stride, stream=None):
    check(load().spb_sparse_ternary_unpack(_p(meta), _p(values), _p(out), rows, cols, meta_row_stride,
                                           values_row_stride, _stream(stream)))


def sparse_ternary_gemv_gpu(meta, values, x, y, rows, cols, meta_row_stride, values_row_stride, stream=None):
    check(load().spb_sparse_ternary_gemv(_p(meta), _p(values), _p(x), _p(y), rows, cols, meta_row_stride,
                                         values_row_stride, _stream(stream)))


def prepared_weights_bytes(rows, cols) -> int:
    return int(load().spb_prepared_weights_bytes(rows, cols))


def prepare_weights(meta, values, rows, cols, meta_row_stride, values_row_stride, stream=None):
    """Packed rows on the device -> the prepared form (a uint8 CUDA tensor) that prepared_gemv_gpu takes."""
    nbytes = prepared_weights_bytes(rows, cols)
    if nbytes == 0:
        raise ValueError(f"prepared weights: shape {rows}x{cols} not taken (cols must be a multiple of 256)")
    out = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    check(load().spb_prepare_weights(_p(meta), _p(values), rows, cols, meta_row_stride, values_row_stride, _p(out),
                                     _stream(stream)))
    return out


def prepared_gemv_gpu(prepared, x, y, rows, cols, stream=None):
    check(load().spb_prepared_gemv(_p(prepared), _p(x), _p(y), rows, cols, _stream(stream)))


def prepared_bitlinear_q8_gpu(prepared, xq, out_half, d_absmax, gamma, rows, cols, stream=None):
    check(load().spb_prepared_bitlinear_q8(_p(prepared), _p(xq), _p(out_half), _p(d_absmax), float(gamma), rows, cols,
                                           _stream(stream)))


class GemvWorkList:
    """A device-resident list of GEMVs for sparse_ternary_gemv_batch_gpu.  items: iterable of
    (meta, values, x, y, rows, cols, meta_row_stride, values_row_stride) with CUDA tensors (or
    device addresses) for the first four."""

    def __init__(self, items):
        import numpy as np
        from ._lib import GemvItem
        items = list(items)
        arr = (GemvItem * len(items))()
        for i, (meta, values, x, y, rows, cols, ms, vs) in enumerate(items):
            arr[i] = GemvItem(_p(meta).value, _p(values).value, _p(x).value, _p(y).value, rows, cols, ms, vs)
        check(load().spb_gemv_batch_check(arr, len(items)))
        self.n = len(items)
        self.max_rows = max((it[4] for it in items), default=0)
        self.max_cols = max((it[5] for it in items), default=0)
        raw = np.frombuffer(bytes(arr), dtype=np.uint8).copy() if items else np.zeros(1, np.uint8)
        self.d_items = torch.from_numpy(raw).cuda()
        self._keep = items  # keeps the tensors alive


def sparse_ternary_gemv_batch_gpu(work: GemvWorkList, stream=None):
    check(load().spb_sparse_ternary_gemv_batch(_p(work.d_items), work.n, work.max_rows, work.max_cols,
                                               _stream(stream)))


def sparse_ternary_gemv_scaled_gpu(meta, values, x, y, y_acc, d_absmax, gamma, rows, cols, meta_row_stride,
                                   values_row_stride, stream=None):
    check(load().spb_sparse_ternary_gemv_scaled(_p(meta), _p(values), _p(x), _p(y), _p(y_acc), _p(d_absmax),
                                                float(gamma), rows, cols, meta_row_stride, values_row_stride,
                                                _stream(stream)))


def fused_sparse_bitlinear_gpu(meta, values, x, output, d_absmax, gamma, rows, cols, meta_row_stride,
                               values_row_stride, stream=None):
    check(load().spb_fused_sparse_bitlinear(_p(meta), _p(values), _p(x), _p(output), _p(d_absmax), float(gamma),
                                            rows, cols, meta_row_stride, values_row_stride, _stream(stream)))


def sparse_bitlinear_q8_gpu(meta, values, xq, output, d_absmax, gamma, rows, cols, meta_row_stride,
                            values_row_stride, stream=None):
    check(load().spb_sparse_bitlinear_q8(_p(meta), _p(values), _p(xq), _p(output), _p(d_absmax), float(gamma),
                                         rows, cols, meta_row_stride, values_row_stride, _stream(stream)))


def sparse_ternary_gemm_gpu(meta, values, X, Y, rows, cols, n, meta_row_stride, values_row_stride, stream=None):
    check(load().spb_sparse_ternary_gemm(_p(meta), _p(values), _p(X), _p(Y), rows, cols, n, meta_row_stride,
                                         values_row_stride, _stream(stream)))


def sparse_bitlinear_gemm_gpu(meta, values, Xq, output, d_absmax, gamma, rows, cols, n, meta_row_stride,
                              values_row_stride, acc_workspace=None, stream=None):
    """BitLinear over n quantised activation rows (no counterpart in the reference, whose prefill is token-serial):
    output[j] = half(float(W @ Xq[j]) * (gamma * d_absmax[j] / 127)).  acc_workspace: n * rows int32, needed only by
    the forms without a fused epilogue."""
    ws = _p(acc_workspace) if acc_workspace is not None else None
    check(load().spb_sparse_bitlinear_gemm(_p(meta), _p(values), _p(Xq), _p(output), _p(d_absmax), float(gamma), ws,
                                           rows, cols, n, meta_row_stride, values_row_stride, _stream(stream)))


# ---- inference_kernels.h ----------------------------------------------------------------

def rms_norm_gpu(input, weight, output, size, eps, stream=None):
    check(load().spb_rms_norm(_p(input), _p(weight), _p(output), size, float(eps), _stream(stream)))


def absmax_quantize_gpu(input, output, d_absmax, size, stream=None):
    check(load().spb_absmax_quantize(_p(input), _p(output), _p(d_absmax), size, _stream(stream)))


def absmax_reduce_gpu(input, d_absmax, size, stream=None):
    check(load().spb_absmax_reduce(_p(input), _p(d_absmax), size, _stream(stream)))


def dequantize_gpu(input, output, d_absmax, gamma, size, stream=None):
    check(load().spb_dequantize(_p(input), _p(output), _p(d_absmax), float(gamma), size, _stream(stream)))


def rope_gpu(vec, num_heads, head_dim, pos, theta, stream=None):
    check(load().spb_rope(_p(vec), num_heads, head_dim, pos, float(theta), _stream(stream)))


def scatter_kv_gpu(src, cache, num_kv_heads, head_dim, max_seq_len, pos, stream=None):
    check(load().spb_scatter_kv(_p(src), _p(cache), num_kv_heads, head_dim, max_seq_len, pos, _stream(stream)))


def attention_scores_gpu(Q, K_cache, scores, num_heads, num_kv_heads, head_dim, max_seq_len, seq_len, scale,
                         stream=None):
    check(load().spb_attention_scores(_p(Q), _p(K_cache), _p(scores), num_heads, num_kv_heads, head_dim,
                                      max_seq_len, seq_len, float(scale), _stream(stream)))


def softmax_gpu(scores, num_heads, max_seq_len, seq_len, stream=None):
    check(load().spb_softmax(_p(scores), num_heads, max_seq_len, seq_len, _stream(stream)))


def attention_output_gpu(scores, V_cache, output, num_heads, num_kv_heads, head_dim, max_seq_len, seq_len,
                         stream=None):
    check(load().spb_attention_output(_p(scores), _p(V_cache), _p(output), num_heads, num_kv_heads, head_dim,
                                      max_seq_len, seq_len, _stream(stream)))


def decode_attention_gpu(Q, K_cache, V_cache, output, num_heads, num_kv_heads, head_dim, max_seq_len, seq_len,
                         scale, stream=None):
    check(load().spb_decode_attention(_p(Q), _p(K_cache), _p(V_cache), _p(output), num_heads, num_kv_heads,
                                      head_dim, max_seq_len, seq_len, float(scale), _stream(stream)))


def decode_attention_scratch_bytes(num_heads, head_dim, max_seq_len) -> int:
    return int(load().spb_decode_attention_scratch_bytes(num_heads, head_dim, max_seq_len))


def decode_attention_split_gpu(Q, K_cache, V_cache, output, num_heads, num_kv_heads, head_dim, max_seq_len, seq_len,
                               scale, scratch, stream=None):
    nbytes = scratch.numel() * scratch.element_size()
    check(load().spb_decode_attention_split(_p(Q), _p(K_cache), _p(V_cache), _p(output), num_heads, num_kv_heads,
                                            head_dim, max_seq_len, seq_len, float(scale), _p(scratch), nbytes,
                                            _stream(stream)))


def relu2_mul_gpu(gate, up, output, size, stream=None):
    check(load().spb_relu2_mul(_p(gate), _p(up), _p(output), size, _stream(stream)))


def relu2_mul_f32_gpu(gate, up, output, size, stream=None):
    check(load().spb_relu2_mul_f32(_p(gate), _p(up), _p(output), size, _stream(stream)))


def rms_norm_f32in_gpu(input, weight, output, size, eps, stream=None):
    check(load().spb_rms_norm_f32in(_p(input), _p(weight), _p(output), size, float(eps), _stream(stream)))


def float_to_half_gpu(input, output, size, stream=None):
    check(load().spb_float_to_half(_p(input), _p(output), size, _stream(stream)))


def residual_add_gpu(a, b, output, size, stream=None):
    check(load().spb_residual_add(_p(a), _p(b), _p(output), size, _stream(stream)))


def half_gemv_gpu(W, x, y, rows, cols, stream=None):
    check(load().spb_half_gemv(_p(W), _p(x), _p(y), rows, cols, _stream(stream)))


# ---- conversion on the GPU (no counterpart among the reference's GPU wrappers) -----------------

def prune_pack_gpu(weights, stream=None):
    """Magnitude 2:4 pruning + sign extraction + packing of a CUDA float32 matrix, byte-identical to
    python/convert_model.py (generate_24_mask, quantize_ternary_absmean, the zero-at-mask fix,
    pack_sparse_ternary).  Returns (meta, values, gamma): int32 CUDA tensors holding the uint32 words,
    and gamma = mean |w| accumulated in double precision."""
    import torch
    assert weights.is_cuda and weights.dtype == torch.float32 and weights.dim() == 2 and weights.stride(1) == 1
    rows, cols = weights.shape
    ms, vs = (cols // 4 + 7) // 8, (cols // 4 + 15) // 16
    meta = torch.zeros((rows, ms), dtype=torch.int32, device=weights.device)
    values = torch.zeros((rows, vs), dtype=torch.int32, device=weights.device)
    abs_sum = torch.zeros(1, dtype=torch.float64, device=weights.device)
    check(load().spb_prune_pack_gpu(_p(weights), rows, cols, weights.stride(0), _p(meta), _p(values), ms, vs,
                                    _p(abs_sum), _stream(stream)))
    gamma = float(abs_sum.item()) / max(1, rows * cols)
    return meta, values, gamma
