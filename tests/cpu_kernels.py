"""CPU stand-ins for the per-op entry points of spbitnet_b200.kernels that sharding.ShardedEngine calls, built on the
oracle (test infrastructure only): same names and argument order, torch CPU tensors instead of device tensors.  They
let the sharded decode step - its row split, its all-gathers and its op order - run under a gloo process group
without a GPU."""
import numpy as np
import torch

import oracle


def _np16(t, n=None):
    a = t.detach().numpy()
    return a.reshape(-1)[: a.size if n is None else n]


def _put16(dst, values):
    dst.view(-1)[: values.size] = torch.from_numpy(np.ascontiguousarray(values).view(np.int16)).view(torch.float16)


def rms_norm_gpu(input, weight, output, size, eps, stream=None):
    _put16(output, oracle.rms_norm(_np16(input, size), weight.numpy(), eps))


def absmax_quantize_gpu(input, output, d_absmax, size, stream=None):
    q, a = oracle.absmax_quantize(_np16(input, size))
    output.view(-1)[:size] = torch.from_numpy(q)
    d_absmax[0] = float(a)


def sparse_bitlinear_q8_gpu(meta, values, xq, output, d_absmax, gamma, rows, cols, meta_row_stride, values_row_stride,
                            stream=None):
    m = meta.numpy().view(np.uint32).reshape(rows, meta_row_stride)
    v = values.numpy().view(np.uint32).reshape(rows, values_row_stride)
    acc = oracle.sparse_gemv(m, v, xq.numpy().reshape(-1)[:cols], rows, cols)
    _put16(output, oracle.dequantize(acc, np.float32(d_absmax[0].item()), np.float32(gamma)))


def rope_gpu(vec, num_heads, head_dim, pos, theta, stream=None):
    _put16(vec, oracle.rope(_np16(vec, num_heads * head_dim), num_heads, head_dim, pos, theta))


def scatter_kv_gpu(src, cache, num_kv_heads, head_dim, max_seq_len, pos, stream=None):
    _put16(cache, oracle.scatter_kv(_np16(src, num_kv_heads * head_dim), _np16(cache), num_kv_heads, head_dim,
                                    max_seq_len, pos))


def decode_attention_gpu(Q, K_cache, V_cache, output, num_heads, num_kv_heads, head_dim, max_seq_len, seq_len, scale,
                         stream=None):
    _put16(output, oracle.attention(_np16(Q, num_heads * head_dim), _np16(K_cache), _np16(V_cache), num_heads,
                                    num_kv_heads, head_dim, max_seq_len, seq_len, scale))


def residual_add_gpu(a, b, output, size, stream=None):
    _put16(output, oracle.residual_add(_np16(a, size), _np16(b, size)))


def relu2_mul_f32_gpu(gate, up, output, size, stream=None):
    output.view(-1)[:size] = torch.from_numpy(oracle.relu2_mul_f32(_np16(gate, size), _np16(up, size)))


def rms_norm_f32in_gpu(input, weight, output, size, eps, stream=None):
    _put16(output, oracle.rms_norm_f32in(input.numpy().reshape(-1)[:size], weight.numpy(), eps))


def float_to_half_gpu(input, output, size, stream=None):
    _put16(output, oracle.float_to_half(input.numpy().reshape(-1)[:size]))


def half_gemv_gpu(W, x, y, rows, cols, stream=None):
    y.view(-1)[:rows] = torch.from_numpy(oracle.half_gemv(W.numpy()[:rows], _np16(x, cols)))
